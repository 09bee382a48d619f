"""No GPU needed: the shared library loads, exports every symbol the headers
declare, and the structs have the binary layout of the reference's types.h."""
import ctypes as C
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


def _declared_functions():
    names = set()
    for rel in ("tensorfuse/tensorfuse.h", "tensorfuse_b200.h"):
        src = open(os.path.join(INC, rel)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", src):
            n = m.group(1)
            if n.startswith(("tensorfuse_", "fused_", "optimized_")) and not n.endswith(("sizeof_dtype", "size_bytes")):
                names.add(n)
    return names


def test_library_exports_every_declared_symbol():
    from tensorfuse_b200._lib import LIB_PATH
    lib = C.CDLL(LIB_PATH)
    names = _declared_functions()
    assert len(names) >= 35
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing
    # C++ symbols the reference's tests look up by mangled name
    for n in ("_ZN10tensorfuse7kernels25fused_gemm_bias_gelu_fp32EPKvS2_S2_PviiiffP11CUstream_st",
              "_ZN10tensorfuse7kernels25fused_gemm_bias_gelu_fp16EPKvS2_S2_PviiiffP11CUstream_st"):
        assert hasattr(lib, n)


def test_struct_layout_matches_reference_abi(tmp_path):
    from tensorfuse_b200._lib import Config, Shape, Tensor
    # sizes/offsets measured from the reference's src/tensorfuse/types.h with gcc (x86-64)
    assert C.sizeof(Shape) == 68 and C.sizeof(Tensor) == 120 and C.sizeof(Config) == 40
    assert (Tensor.dtype.offset, Tensor.size_bytes.offset, Tensor.scale.offset) == (76, 88, 104)
    # and the C header of this repo agrees with the ctypes mirror
    prog = tmp_path / "abi.c"
    prog.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "tensorfuse/tensorfuse.h"\n'
                    '#include "tensorfuse_b200.h"\n'
                    'int main(){printf("%zu %zu %zu %zu %zu %zu %d %d", sizeof(TensorFuseShape), sizeof(TensorFuseTensor),'
                    'offsetof(TensorFuseTensor,dtype), offsetof(TensorFuseTensor,scale), sizeof(TensorFuseConfig),'
                    'sizeof(TensorFuseTransformerParams), (int)TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE, (int)TENSORFUSE_INT32);return 0;}')
    exe = tmp_path / "abi"
    subprocess.run(["gcc", "-std=c11", "-I", INC, str(prog), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    assert out == ["68", "120", "76", "104", "40", "152", "11", "5"]


def test_status_codes_without_a_device():
    """On a machine without a GPU init reports a CUDA error and every operator
    refuses to run: there is no CPU fallback."""
    import torch
    if torch.cuda.is_available():
        return
    from tensorfuse_b200._lib import Tensor, lib
    assert lib.tensorfuse_init(None) == 2
    t = Tensor()
    assert lib.tensorfuse_fused_gemm_bias_gelu(C.byref(t), C.byref(t), C.byref(t), C.byref(t), None) == 4
    assert lib.tensorfuse_fused_softmax_dropout(C.byref(t), C.byref(t), None, 0.0, None) == 4
    assert lib.tensorfuse_b200_gemm_bias_gelu_host(None, None, None, None, 1, 1, 1, 0, 0, 0, 0, 1.0, 1.0) == 4
    assert lib.tensorfuse_get_error_string(4) == b"Library not initialized"
    assert lib.tensorfuse_shutdown() == 0


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "tensorfuse_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f in ("softmax_dropout.cu", "kernels.h"), (dirpath, f)
    code = "import sys; import tensorfuse_b200; assert not any(m.startswith('oracle') for m in sys.modules)"
    subprocess.run([sys.executable, "-c", code], check=True, cwd=ROOT)
