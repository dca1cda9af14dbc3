"""Generates tests/golden/fingerprints.json from the REFERENCE's own host code.

Runs only where the reference tree is mounted (the REF path below, the default of oracle/Makefile): it loads oracle/_ref/libref_host.so, which oracle/Makefile
(`make -C oracle ref`) compiles from the reference's unmodified src/set_ops, src/fingerprint and
src/datatype sources, calls the reference's set_native_*_skeleton builders for every (op, datatype)
identity its register_native_ops enumerates, and records nickname, argument datatypes and SHA-256
fingerprint, plus datatype names/sizes and the sizeof/offsetof table of the ABI structs (abi_layout.c compiled
against the reference's headers). The committed JSON is what the CPU tests
compare this library's registry against.

    make -C oracle ref && python tests/golden/make_fingerprints.py
"""
import ctypes as C
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_host.so"))


class Header(C.Structure):
    _fields_ = [("op_nickname", C.c_char * 256), ("num_args", C.c_int), ("arg_dtypes", C.c_int * 32)]


class Skeleton(C.Structure):
    _fields_ = [("header", Header), ("fingerprint", C.c_uint8 * 32)]


ref.set_native_op_skeleton.argtypes = [C.POINTER(Skeleton), C.c_char_p, C.c_int, C.c_int]
ref.dataflow_datatype_as_string.restype = C.c_char_p
ref.dataflow_datatype_as_string.argtypes = [C.c_int]
ref.dataflow_sizeof_element.restype = C.c_size_t
ref.dataflow_sizeof_element.argtypes = [C.c_int]

FP32, FP16, BF16, E4M3, E5M2 = 3, 4, 5, 6, 7
FWD = [FP32, FP16, BF16, E4M3, E5M2]
BWD = [FP32, FP16, BF16]
PAIRS = [(FP32, FP32), (FP16, FP16), (BF16, BF16), (E4M3, FP16), (E4M3, BF16), (E5M2, FP16), (E5M2, BF16)]
FAMILIES = {  # op -> list of (fwd_dt, bwd_dt) as the reference's register_native_ops passes them
    "embedding": [(f, 0) for f in FWD], "rms_norm": [(f, 0) for f in FWD], "rope": [(f, 0) for f in FWD],
    "swiglu": [(f, 0) for f in FWD], "copy_to_seq_context": [(f, 0) for f in FWD],
    "rms_norm_bwd_x": PAIRS, "rms_norm_bwd_w": PAIRS, "swiglu_bwd_x": PAIRS, "softmax": PAIRS,
    "rope_bwd_x": [(0, b) for b in BWD], "cross_entropy_loss": [(0, b) for b in BWD],
}

records = []
for op, variants in FAMILIES.items():
    for fwd, bwd in variants:
        sk = Skeleton()
        C.memset(C.byref(sk), 0xAB, C.sizeof(sk))      # the builders must define every byte they hash
        assert ref.set_native_op_skeleton(C.byref(sk), op.encode(), fwd, bwd) == 0
        records.append({"op": op, "fwd_dt": fwd, "bwd_dt": bwd, "nickname": sk.header.op_nickname.decode(),
                        "num_args": sk.header.num_args, "arg_dtypes": list(sk.header.arg_dtypes),
                        "fingerprint": bytes(sk.fingerprint).hex()})

# struct layouts, from the reference's own headers
import subprocess
import tempfile
REF = os.environ.get("REF", "/root/reference")          # the reference tree, as in oracle/Makefile (REF ?= ...)
inc = [f"-I{REF}/include", f"-I{REF}/src/datatype/include", f"-I{REF}/src/table/include", f"-I{REF}/src/ops/include",
       f"-I{REF}/src/dataflow_handle/include", f"-I{REF}/src/dataflow_handle/nvidia/include", "-I/usr/local/cuda/include"]
with tempfile.TemporaryDirectory() as td:
    exe = os.path.join(td, "abi_layout")
    subprocess.check_call(["gcc", "-DUSE_REFERENCE_HEADERS", "-w", *inc, os.path.join(HERE, "abi_layout.c"), "-o", exe])
    layout = json.loads(subprocess.check_output([exe]))

out = {
    "layout": layout,
    "source": "als244/dataflow_lib src/set_ops/src/set_native_op_skeletons.c via oracle/_ref/libref_host.so",
    "sizeof": {"Op_Skeleton_Header": C.sizeof(Header), "Op_Skeleton": C.sizeof(Skeleton), "Op": C.sizeof(Skeleton) + 8 * 32},
    "datatype_names": {str(i): ref.dataflow_datatype_as_string(i).decode() for i in range(28)},
    "datatype_sizes": {str(i): ref.dataflow_sizeof_element(i) for i in range(28)},
    "skeletons": records,
}
with open(os.path.join(HERE, "fingerprints.json"), "w") as f:
    json.dump(out, f, indent=1)
print(f"wrote {len(records)} skeletons")
