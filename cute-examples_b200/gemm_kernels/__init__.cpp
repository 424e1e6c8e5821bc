// PyTorch binding of the sm_100a TN GEMM: module gemm_kernels._C.
// Same module name, function name, argument names and order as the reference's binding
// (kernels/gemm_kernels/__init__.cpp:6-9): gemm_tn_test(A, B, C) writes A * B^T into the
// caller's C and returns that same tensor (kernels/gemm_kernels/sm90a/gemm_test.cu:91).
// All device work happens behind the C ABI of include/gemm_sm100.h; this file only checks
// tensors and hands over pointers, sizes and the current stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/gemm_sm100.h"

namespace test {

namespace {

void raise_for(int rc, int cuda_error, const char* what) {
  if (rc == GEMM_SM100_OK) return;
  std::string msg = std::string(what) + ": " + gemm_sm100_error_string(rc);
  if (rc == GEMM_SM100_ERR_CUDA) msg += " (cudaError_t " + std::to_string(cuda_error) + ")";
  TORCH_CHECK(false, msg);
}

int dtype_code(const torch::Tensor& t) {
  if (t.scalar_type() == torch::kBFloat16) return GEMM_SM100_BF16;
  if (t.scalar_type() == torch::kFloat16) return GEMM_SM100_FP16;
  TORCH_CHECK(false, "Both tensors must be of type bfloat16 or float16");
  return -1;
}

// K-split scratch memory, kept between calls: one buffer per (device, stream), grown on demand.
// A torch::empty per call costs microseconds, which is a large part of the few-tile, long-K
// GEMMs that use the schedule.  Keyed by stream because two GEMMs on different streams may run at
// the same time and must not share partial tiles; calls on one stream are ordered.  The
// buffers come from torch's caching allocator and live until the process ends.
void* kept_workspace(const c10::Device& device, cudaStream_t stream, size_t bytes) {
  static std::mutex mutex;
  static std::map<std::pair<int, cudaStream_t>, torch::Tensor> kept;
  std::lock_guard<std::mutex> lock(mutex);
  torch::Tensor& t = kept[{static_cast<int>(device.index()), stream}];
  if (!t.defined() || static_cast<size_t>(t.numel()) < bytes) {
    // the old buffer (if any) goes back to the allocator, which keeps it alive for the work
    // already queued on the stream it was allocated on
    if (t.defined()) gemm_sm100_workspace_unregister(t.data_ptr());
    t = torch::empty({static_cast<int64_t>(bytes)}, torch::TensorOptions().dtype(torch::kUInt8).device(device));
    // kept by the library from here on: zero-filled once, no memset in front of the even K-split
    int cuda_error = 0;
    const int rc = gemm_sm100_workspace_register(t.data_ptr(), bytes, static_cast<void*>(stream), &cuda_error);
    TORCH_CHECK(rc == GEMM_SM100_OK, "gemm_sm100_workspace_register: ", gemm_sm100_error_string(rc), " cuda=", cuda_error);
  }
  return t.data_ptr();
}

}  // namespace

// Checks follow the reference's order and wording where it has them (gemm_test.cu:15-41);
// C is checked as well (the reference assumes it), tile-divisibility is not required.
torch::Tensor gemm_tn_test(const torch::Tensor A, const torch::Tensor B, torch::Tensor C) {
  // Shape and dtype first (these need no device), then placement.
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "Both tensors must be 2D (matrix) tensors");
  // The reference insists on contiguous operands (gemm_test.cu:18-19); rows with a larger pitch
  // are accepted here as long as K stays contiguous.
  TORCH_CHECK((A.numel() == 0 || A.stride(1) == 1) && (B.numel() == 0 || B.stride(1) == 1),
              "All tensors must be contiguous along K");
  TORCH_CHECK(A.size(1) == B.size(1), "Inner dimensions of A and B must match (A: ", A.size(1),
              ", B: ", B.size(1), ")");
  const int dtype = dtype_code(A);
  TORCH_CHECK(B.scalar_type() == A.scalar_type() && C.scalar_type() == A.scalar_type(),
              "A, B and C must have the same dtype");
  TORCH_CHECK(C.dim() == 2 && C.size(0) == A.size(0) && C.size(1) == B.size(0),
              "C must be a 2D tensor of shape [A.size(0), B.size(0)]");
  TORCH_CHECK(C.numel() == 0 || C.stride(1) == 1, "C must have unit stride along its last dimension");
  TORCH_CHECK(A.size(0) <= INT32_MAX && B.size(0) <= INT32_MAX && A.size(1) <= INT32_MAX,
              "extents must fit in 32 bits");
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda(), "All tensors must be CUDA tensors");
  TORCH_CHECK(A.device() == B.device() && A.device() == C.device(),
              "All tensors must be on the same device");
  const int M = static_cast<int>(A.size(0));
  const int N = static_cast<int>(B.size(0));
  const int K = static_cast<int>(A.size(1));
  if (M == 0 || N == 0) return C;

  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream(A.device().index()).stream();
  const size_t ws_bytes = gemm_sm100_workspace_bytes(M, N, K, dtype);
  void* const ws_ptr = ws_bytes > 0 ? kept_workspace(A.device(), stream, ws_bytes) : nullptr;
  const long ldc = M > 1 ? static_cast<long>(C.stride(0)) : static_cast<long>(N);
  const long lda = M > 1 ? static_cast<long>(A.stride(0)) : static_cast<long>(K);
  const long ldb = N > 1 ? static_cast<long>(B.stride(0)) : static_cast<long>(K);
  int cuda_error = 0;
  int rc;
  {
    pybind11::gil_scoped_release release;
    rc = gemm_sm100_tn(A.const_data_ptr(), B.const_data_ptr(), C.mutable_data_ptr(), M, N, K,
                       lda, ldb, ldc, dtype, ws_ptr, ws_bytes,
                       static_cast<void*>(stream), &cuda_error);
  }
  raise_for(rc, cuda_error, "gemm_tn_test");
  return C;
}

// C[M,N] = op(A) * op(B) for the four operand layouts: A as [M,K] or [K,M] (a_is_km), B as [N,K] or
// [K,N] (b_is_kn).  No transposed copies are made; the [K,*] forms go to the tensor core as
// MN-major operands.
torch::Tensor gemm_layouts(const torch::Tensor A, const torch::Tensor B, torch::Tensor C, bool a_is_km,
                           bool b_is_kn, double alpha = 1.0, double beta = 0.0) {
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2, "All tensors must be 2D (matrix) tensors");
  TORCH_CHECK((A.numel() == 0 || A.stride(1) == 1) && (B.numel() == 0 || B.stride(1) == 1) &&
                  (C.numel() == 0 || C.stride(1) == 1),
              "All tensors must have unit stride along their last dimension");
  const int64_t M = a_is_km ? A.size(1) : A.size(0);
  const int64_t Ka = a_is_km ? A.size(0) : A.size(1);
  const int64_t N = b_is_kn ? B.size(1) : B.size(0);
  const int64_t Kb = b_is_kn ? B.size(0) : B.size(1);
  TORCH_CHECK(Ka == Kb, "Inner dimensions of A and B must match (A: ", Ka, ", B: ", Kb, ")");
  const int dtype = dtype_code(A);
  TORCH_CHECK(B.scalar_type() == A.scalar_type() && C.scalar_type() == A.scalar_type(),
              "A, B and C must have the same dtype");
  TORCH_CHECK(C.size(0) == M && C.size(1) == N, "C must be of shape [", M, ", ", N, "]");
  TORCH_CHECK(M <= INT32_MAX && N <= INT32_MAX && Ka <= INT32_MAX, "extents must fit in 32 bits");
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda(), "All tensors must be CUDA tensors");
  TORCH_CHECK(A.device() == B.device() && A.device() == C.device(), "All tensors must be on the same device");
  if (M == 0 || N == 0) return C;
  if (!a_is_km && !b_is_kn && alpha == 1.0 && beta == 0.0) return gemm_tn_test(A, B, C);
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream(A.device().index()).stream();
  const long lda = A.size(0) > 1 ? static_cast<long>(A.stride(0)) : static_cast<long>(A.size(1));
  const long ldb = B.size(0) > 1 ? static_cast<long>(B.stride(0)) : static_cast<long>(B.size(1));
  const long ldc = M > 1 ? static_cast<long>(C.stride(0)) : static_cast<long>(N);
  int cuda_error = 0;
  int rc;
  {
    pybind11::gil_scoped_release release;
    rc = gemm_sm100_gemm_scaled(A.const_data_ptr(), B.const_data_ptr(), C.mutable_data_ptr(), static_cast<int>(M),
                                static_cast<int>(N), static_cast<int>(Ka), lda, ldb, ldc, dtype, a_is_km ? 1 : 0,
                                b_is_kn ? 1 : 0, static_cast<float>(alpha), static_cast<float>(beta),
                                static_cast<void*>(stream), &cuda_error);
  }
  raise_for(rc, cuda_error, "gemm_layouts");
  return C;
}

torch::Tensor gemm_nn(const torch::Tensor A, const torch::Tensor B, torch::Tensor C) {
  return gemm_layouts(A, B, C, false, true);
}

// A * B^T stored through raw device pointers into several outputs of shape [M, N] with row pitch
// `ldc` (elements).  The pointers may name peer-GPU memory mapped into this process; they are
// not tensors on purpose (symmetric-memory handles expose peers as addresses).
void gemm_tn_fanout(const torch::Tensor A, const torch::Tensor B, const std::vector<int64_t>& output_ptrs,
                    int64_t ldc) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda(), "All tensors must be CUDA tensors");
  TORCH_CHECK(A.device() == B.device(), "All tensors must be on the same device");
  TORCH_CHECK(A.is_contiguous() && B.is_contiguous(), "All tensors must be contiguous");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "Both tensors must be 2D (matrix) tensors");
  TORCH_CHECK(A.size(1) == B.size(1), "Inner dimensions of A and B must match (A: ", A.size(1),
              ", B: ", B.size(1), ")");
  TORCH_CHECK(B.scalar_type() == A.scalar_type(), "A and B must have the same dtype");
  TORCH_CHECK(!output_ptrs.empty() && output_ptrs.size() <= 8, "between 1 and 8 outputs");
  const int dtype = dtype_code(A);
  std::vector<void*> outs;
  for (int64_t ptr : output_ptrs) outs.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(ptr)));
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream(A.device().index()).stream();
  int cuda_error = 0;
  int rc;
  {
    pybind11::gil_scoped_release release;
    rc = gemm_sm100_tn_fanout(A.const_data_ptr(), B.const_data_ptr(), outs.data(), static_cast<int>(outs.size()),
                              static_cast<int>(A.size(0)), static_cast<int>(B.size(0)), static_cast<int>(A.size(1)),
                              static_cast<long>(A.size(1)), static_cast<long>(A.size(1)), static_cast<long>(ldc),
                              dtype, static_cast<void*>(stream), &cuda_error);
  }
  raise_for(rc, cuda_error, "gemm_tn_fanout");
}

// Waits for the current device and raises if a kernel reported a timed-out wait.
unsigned int device_status() {
  unsigned int word = 0;
  int cuda_error = 0;
  int rc;
  {
    pybind11::gil_scoped_release release;
    rc = gemm_sm100_device_status(&word, &cuda_error);
  }
  if (rc == GEMM_SM100_ERR_DEVICE_TIMEOUT) {
    TORCH_CHECK(false, "gemm_sm100: device-side wait timed out, status word 0x", std::hex, word);
  }
  raise_for(rc, cuda_error, "device_status");
  return word;
}

// Registers (or, with an undefined tensor, removes) the device buffer the kernels write their
// per-CTA trace records to; see gemm_sm100_set_trace_buffer.
void set_trace_buffer(const c10::optional<torch::Tensor>& buffer) {
  if (!buffer.has_value()) {
    raise_for(gemm_sm100_set_trace_buffer(nullptr, 0), 0, "set_trace_buffer");
    return;
  }
  const torch::Tensor& t = buffer.value();
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kInt64,
              "trace buffer must be a contiguous CUDA int64 tensor");
  raise_for(gemm_sm100_set_trace_buffer(t.data_ptr(), static_cast<size_t>(t.numel()) * 8), 0, "set_trace_buffer");
}

// One-time set-up of the current device (see gemm_sm100_init); optional.
void init() {
  int cuda_error = 0;
  raise_for(gemm_sm100_init(&cuda_error), cuda_error, "init");
}

void set_option(const std::string& name, long value) {
  raise_for(gemm_sm100_set_option(name.c_str(), value), 0, "set_option");
}

std::string describe_config(int index) {
  char buf[256];
  raise_for(gemm_sm100_describe_config(index, buf, sizeof(buf)), 0, "describe_config");
  return std::string(buf);
}

std::string describe_plan(int M, int N, int K, int dtype) {
  char buf[384];
  raise_for(gemm_sm100_describe_plan(M, N, K, dtype, buf, sizeof(buf)), 0, "describe_plan");
  return std::string(buf);
}

PYBIND11_MODULE(_C, m) {
  m.def("gemm_tn_test", &gemm_tn_test, "GEMM transpose-normal test function", pybind11::arg("A"),
        pybind11::arg("B"), pybind11::arg("C"));
  m.def("gemm_layouts", &gemm_layouts,
        "C = alpha * op(A) * op(B) + beta * C: A as [M,K] or [K,M], B as [N,K] or [K,N]",
        pybind11::arg("A"), pybind11::arg("B"), pybind11::arg("C"), pybind11::arg("a_is_km"), pybind11::arg("b_is_kn"),
        pybind11::arg("alpha") = 1.0, pybind11::arg("beta") = 0.0);
  m.def("gemm_nn", &gemm_nn, "C = A[M,K] * B[K,N] into the caller's C", pybind11::arg("A"), pybind11::arg("B"),
        pybind11::arg("C"));
  m.def("gemm_tn_fanout", &gemm_tn_fanout, "A * B^T stored into several outputs given as device addresses",
        pybind11::arg("A"), pybind11::arg("B"), pybind11::arg("output_ptrs"), pybind11::arg("ldc"));
  m.def("device_status", &device_status,
        "Synchronise the current device and raise if a GEMM kernel reported a failed wait");
  m.def("init", &init, "One-time set-up of the current device; call before capturing a CUDA graph");
  m.def("set_option", &set_option, pybind11::arg("name"), pybind11::arg("value"));
  m.def("set_trace_buffer", &set_trace_buffer, pybind11::arg("buffer"));
  m.def("describe_config", &describe_config, pybind11::arg("index"));
  m.def("describe_plan", &describe_plan, pybind11::arg("M"), pybind11::arg("N"), pybind11::arg("K"),
        pybind11::arg("dtype"));
  m.def("select_config", &gemm_sm100_select_config, pybind11::arg("M"), pybind11::arg("N"),
        pybind11::arg("K"), pybind11::arg("dtype"));
  m.def("workspace_bytes", &gemm_sm100_workspace_bytes, pybind11::arg("M"), pybind11::arg("N"),
        pybind11::arg("K"), pybind11::arg("dtype"));
  m.def("num_sms", &gemm_sm100_num_sms);
}

}  // namespace test
