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
    for rel in ("tensorfuse/tensorfuse.h", "tensorfuse/profiler.h", "tensorfuse_b200.h"):   # the extern "C" headers
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
    # C++ symbols of namespace tensorfuse::kernels: the reference's tests look two of
    # them up by mangled name (src/tests/test_kernels_simple.cpp:62-63) and declare the
    # others inline; all eight are part of the binary interface
    gemm = "EPKvS2_S2_PviiiffP11CUstream_st"
    for n in ("_ZN10tensorfuse7kernels25fused_gemm_bias_gelu_fp32" + gemm,
              "_ZN10tensorfuse7kernels25fused_gemm_bias_gelu_fp16" + gemm,
              "_ZN10tensorfuse7kernels25fused_gemm_bias_gelu_int8" + gemm,
              "_ZN10tensorfuse7kernels37fused_gemm_bias_gelu_int8_with_scalesEPKvS2_S2_PviiiffffP11CUstream_st",
              "_ZN10tensorfuse7kernels35optimized_fused_gemm_bias_gelu_fp32" + gemm,
              "_ZN10tensorfuse7kernels35optimized_fused_gemm_bias_gelu_fp16" + gemm,
              "_ZN10tensorfuse7kernels26fused_softmax_dropout_fp16EPKvPvPhiiiifyP11CUstream_st",
              "_ZN10tensorfuse7kernels26fused_softmax_dropout_fp32EPKvPvPhiiiifyP11CUstream_st"):
        assert hasattr(lib, n), n


def test_cxx_namespace_interface_links(tmp_path):
    """include/tensorfuse.h (reference src/tensorfuse.h:36-246, declared there and
    never defined): a C++ program that names every function of the namespace
    links against the library, and the device-free ones answer."""
    import shutil
    from tensorfuse_b200._lib import LIB_PATH
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")), "include")
    prog = tmp_path / "ns.cpp"
    prog.write_text(r"""
#include <cstdio>
#include <cstring>
#include "tensorfuse.h"
#include "tensorfuse/kernels.h"
#include "tensorfuse_b200.h"
namespace tf = tensorfuse;
int main() {
  // every declaration has a definition: taking the address forces the link
  const void* fns[] = {
    (const void*)&tf::initialize, (const void*)&tf::cleanup, (const void*)&tf::get_context,
    (const void*)&tf::get_device_info, (const void*)&tf::set_random_seed, (const void*)&tf::fused_gemm_bias_gelu,
    (const void*)&tf::fused_softmax_dropout, (const void*)&tf::allocate_device, (const void*)&tf::deallocate_device,
    (const void*)&tf::allocate_host, (const void*)&tf::deallocate_host, (const void*)&tf::copy_host_to_device,
    (const void*)&tf::copy_device_to_host, (const void*)&tf::get_memory_stats, (const void*)&tf::create_stream,
    (const void*)&tf::destroy_stream, (const void*)&tf::synchronize, (const void*)&tf::synchronize_stream,
    (const void*)&tf::get_version, (const void*)&tf::get_build_info, (const void*)&tf::get_error_string,
    (const void*)&tf::is_gpu_supported, (const void*)&tf::get_supported_data_types,
    (const void*)&tf::kernels::fused_gemm_bias_gelu_int8_with_scales, (const void*)&tf::kernels::fused_softmax_dropout_fp16,
    (const void*)&tensorfuse_simple_init, (const void*)&tensorfuse_simple_cleanup};
  for (const void* f : fns) if (!f) return 2;
  if (std::strcmp(tf::get_version(), "1.0.0") != 0) return 3;
  if (std::strcmp(tf::get_error_string(TENSORFUSE_ERROR_NOT_INITIALIZED), "Library not initialized") != 0) return 4;
  tf::DataType dt = TENSORFUSE_FLOAT16;
  // not initialised: the operators refuse before touching a pointer
  if (tf::fused_gemm_bias_gelu(nullptr, nullptr, nullptr, nullptr, 1, 1, 1, dt) != TENSORFUSE_ERROR_NOT_INITIALIZED) return 5;
  if (tf::fused_softmax_dropout(nullptr, nullptr, nullptr, 1, 1, 1, 1, 0.0f, dt) != TENSORFUSE_ERROR_NOT_INITIALIZED) return 6;
  if (tf::get_context().is_initialized()) return 7;
  std::printf("%s\n", tf::get_build_info());
  return 0;
}
""")
    exe = tmp_path / "ns"
    libdir = os.path.dirname(LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-I", INC, "-I", cuda_inc, str(prog), "-o", str(exe), "-L", libdir,
                    "-ltensorfuse", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "sm_100a" in r.stdout


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


def test_profiler_helpers_measure_something(tmp_path):
    """Host-side helpers of tensorfuse/profiler.h (placeholders in the reference,
    src/tensorfuse_c_api.cpp:462-643): timers and the roofline arithmetic need no GPU."""
    import time
    from tensorfuse_b200._lib import LIB_PATH

    class Timer(C.Structure):
        _fields_ = [("start_time", C.c_double), ("end_time", C.c_double), ("running", C.c_bool)]

    class Roofline(C.Structure):
        _fields_ = [(n, C.c_float) for n in ("peak_flops", "peak_bandwidth", "arithmetic_intensity", "achieved_flops",
                                             "achieved_bandwidth", "efficiency_flops", "efficiency_bandwidth")] + \
                   [("is_compute_bound", C.c_bool), ("is_memory_bound", C.c_bool)]

    lib = C.CDLL(LIB_PATH)
    lib.tensorfuse_timer_elapsed_ms.restype = C.c_double
    t = Timer()
    lib.tensorfuse_timer_start(C.byref(t)); time.sleep(0.02); lib.tensorfuse_timer_stop(C.byref(t))
    assert 15.0 < lib.tensorfuse_timer_elapsed_ms(C.byref(t)) < 500.0
    lib.tensorfuse_calculate_roofline.argtypes = [C.c_size_t, C.c_size_t, C.c_float, C.POINTER(Roofline)]
    r = Roofline()
    # config 2: 137.44 GFLOP over 176.2 MB in 0.1 ms
    assert lib.tensorfuse_calculate_roofline(137438953472, 176168960, 0.1, C.byref(r)) == 0
    assert r.is_compute_bound and not r.is_memory_bound and abs(r.achieved_flops / 1.374e15 - 1) < 1e-3
    assert abs(r.efficiency_flops - 61.08) < 0.1
    assert lib.tensorfuse_calculate_roofline(1, 1, 0.1, None) == 1
    rid = lib.tensorfuse_profiler_start_region(b"step", b"test")
    assert rid >= 1 and lib.tensorfuse_profiler_end_region(rid) == 0 and lib.tensorfuse_profiler_end_region(10 ** 6) == 1
    out = tmp_path / "prof.json"
    assert lib.tensorfuse_profiler_save(str(out).encode(), b"json") == 0
    import json
    assert json.load(open(out))["regions"][-1]["name"] == "step"
    assert lib.tensorfuse_profiler_reset() == 0
