"""The C++ `namespace tensorfuse` interface (include/tensorfuse.h; reference
src/tensorfuse.h:36-246, which declares it and never defines it) exercised by
a C++ program compiled here and run on the GPU: initialisation, memory and
stream helpers, both operators with the namespace's own argument order, checked
inside the program against the reference's CPU loops
(reference src/tests/test_kernels.cu:43-64, test_softmax_dropout.cu:36-64)."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include <cmath>
#include <cstdio>
#include <vector>
#include "tensorfuse.h"
namespace tf = tensorfuse;

static float gelu_ref(float x) {
  return 0.5f * x * (1.0f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
#define CHECK(cond) do { if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); return 1; } } while (0)

int main() {
  CHECK(tf::is_gpu_supported());
  CHECK(tf::initialize(-1) == TENSORFUSE_SUCCESS);
  CHECK(tf::initialize(-1) == TENSORFUSE_SUCCESS);                 // idempotent
  CHECK(tf::get_context().is_initialized());
  const tf::DeviceInfo info = tf::get_device_info();
  CHECK(info.compute_capability_major == 10 && info.multiprocessor_count > 0 && info.supports_fp8);
  CHECK(tf::get_supported_data_types().size() == 5);

  // GEMM: 37 x 24 x 40 FP32 (not a tile multiple), alpha 0.5, beta 2
  const int M = 37, N = 24, K = 40;
  std::vector<float> A(M * K), B(K * N), bias(N), C(M * N), ref(M * N);
  for (int i = 0; i < M * K; ++i) A[i] = std::sin(0.37f * i);
  for (int i = 0; i < K * N; ++i) B[i] = std::cos(0.11f * i) * 0.3f;
  for (int i = 0; i < N; ++i) bias[i] = 0.01f * i - 0.1f;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float s = 0.0f;
      for (int k = 0; k < K; ++k) s += A[m * K + k] * B[k * N + n];
      ref[m * N + n] = gelu_ref(0.5f * s + 2.0f * bias[n]);
    }
  cudaStream_t stream = tf::create_stream();
  CHECK(stream != nullptr);
  float* dA = (float*)tf::allocate_device(A.size() * 4);
  float* dB = (float*)tf::allocate_device(B.size() * 4, 1024);
  float* db = (float*)tf::allocate_device(bias.size() * 4);
  float* dC = (float*)tf::allocate_device(C.size() * 4);
  CHECK(dA && dB && db && dC && ((size_t)dB % 1024) == 0);
  CHECK(tf::get_memory_stats().num_blocks == 4);
  CHECK(tf::copy_host_to_device(dA, A.data(), A.size() * 4, stream) == TENSORFUSE_SUCCESS);
  CHECK(tf::copy_host_to_device(dB, B.data(), B.size() * 4, stream) == TENSORFUSE_SUCCESS);
  CHECK(tf::copy_host_to_device(db, bias.data(), bias.size() * 4) == TENSORFUSE_SUCCESS);   // synchronous form
  CHECK(tf::fused_gemm_bias_gelu(dA, dB, db, dC, M, N, K, TENSORFUSE_FLOAT32, 0.5f, 2.0f, stream) == TENSORFUSE_SUCCESS);
  CHECK(tf::copy_device_to_host(C.data(), dC, C.size() * 4, stream) == TENSORFUSE_SUCCESS);
  CHECK(tf::synchronize_stream(stream) == TENSORFUSE_SUCCESS);
  float worst = 0.0f;
  for (int i = 0; i < M * N; ++i) worst = std::fmax(worst, std::fabs(C[i] - ref[i]));
  std::printf("gemm max abs error %g\n", worst);
  CHECK(worst < 1e-4f);                                            // reference src/tests/test_kernels.cu:139
  CHECK(tf::fused_gemm_bias_gelu(dA, dB, db, dC, M, N, K, TENSORFUSE_INT32) == TENSORFUSE_ERROR_UNSUPPORTED_OPERATION);

  // softmax: [batch 2, heads 3, seq 5, head_dim 16]; the namespace order is (batch, seq_len, num_heads, head_dim)
  const int Bt = 2, H = 3, S = 5, D = 16, total = Bt * H * S * D;
  std::vector<float> x(total), y(total);
  std::vector<unsigned char> mask(total, 7);
  for (int i = 0; i < total; ++i) x[i] = 2.0f * std::sin(0.73f * i);
  float* dx = (float*)tf::allocate_device(total * 4);
  float* dy = (float*)tf::allocate_device(total * 4);
  unsigned char* dm = (unsigned char*)tf::allocate_device(total);
  CHECK(tf::copy_host_to_device(dx, x.data(), total * 4) == TENSORFUSE_SUCCESS);
  CHECK(tf::fused_softmax_dropout(dx, dy, dm, Bt, S, H, D, 0.0f, TENSORFUSE_FLOAT32, stream) == TENSORFUSE_SUCCESS);
  CHECK(tf::synchronize() == TENSORFUSE_SUCCESS);
  CHECK(tf::copy_device_to_host(y.data(), dy, total * 4) == TENSORFUSE_SUCCESS);
  CHECK(tf::copy_device_to_host(mask.data(), dm, total) == TENSORFUSE_SUCCESS);
  worst = 0.0f;
  for (int r = 0; r < Bt * H * S; ++r) {
    float mx = -INFINITY, sum = 0.0f;
    for (int j = 0; j < D; ++j) mx = std::fmax(mx, x[r * D + j]);
    for (int j = 0; j < D; ++j) sum += std::exp(x[r * D + j] - mx);
    for (int j = 0; j < D; ++j) {
      worst = std::fmax(worst, std::fabs(y[r * D + j] - std::exp(x[r * D + j] - mx) / sum));
      CHECK(mask[r * D + j] == 1);
    }
  }
  std::printf("softmax max abs error %g\n", worst);
  CHECK(worst < 1e-6f);
  CHECK(tf::set_random_seed(11) == TENSORFUSE_SUCCESS);
  CHECK(tf::fused_softmax_dropout(dx, dy, dm, Bt, S, H, D, 1.5f, TENSORFUSE_FLOAT32) == TENSORFUSE_ERROR_INVALID_ARGUMENT);

  void* pinned = tf::allocate_host(4096);
  CHECK(pinned != nullptr);
  tf::deallocate_host(pinned);
  for (void* p : {(void*)dA, (void*)dB, (void*)db, (void*)dC, (void*)dx, (void*)dy, (void*)dm}) tf::deallocate_device(p);
  CHECK(tf::get_memory_stats().num_blocks == 0 && tf::get_memory_stats().peak_usage > 0);
  tf::destroy_stream(stream);
  tf::cleanup();
  CHECK(!tf::get_context().is_initialized());
  CHECK(tf::fused_gemm_bias_gelu(nullptr, nullptr, nullptr, nullptr, 1, 1, 1, TENSORFUSE_FLOAT32) ==
        TENSORFUSE_ERROR_NOT_INITIALIZED);
  std::printf("ALL OK\n");
  return 0;
}
"""


def test_namespace_interface_end_to_end(tmp_path):
    from tensorfuse_b200._lib import LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_root = os.path.dirname(os.path.dirname(nvcc))
    src = tmp_path / "ns_gpu.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "ns_gpu"
    libdir = os.path.dirname(LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda_root, "include"),
                    str(src), "-o", str(exe), "-L", libdir, "-ltensorfuse", f"-Wl,-rpath,{libdir}",
                    "-L", os.path.join(cuda_root, "lib64"), "-lcudart"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ALL OK" in r.stdout, (r.returncode, r.stdout[-2000:], r.stderr[-2000:])
