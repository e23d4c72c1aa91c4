// Torch extension module with the one function the reference's compiled module
// exports: gmm(a, b, c, batch_sizes, trans_a, trans_b) -> None
// (reference: csrc/ops.cu:7-9 binding grouped_gemm::GroupedGemm,
// csrc/grouped_gemm.cu:470-564).  It repeats the reference's argument checks as
// TORCH_CHECKs, takes the current CUDA stream and a workspace from torch's
// caching allocator, and hands raw pointers to the C ABI (include/b200gmm.h).
// All arithmetic lives in libb200gmm.so; nothing here touches the data.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <mutex>
#include <unordered_map>

#include "b200gmm.h"

namespace {

// One status word per device: the kernels OR B200GMM_STATUS_* bits into it.
at::Tensor status_word(const c10::Device& device) {
  static std::mutex mu;
  static std::unordered_map<int, at::Tensor> words;
  std::lock_guard<std::mutex> lock(mu);
  auto it = words.find(device.index());
  if (it == words.end()) {
    it = words.emplace(device.index(),
                       at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(device))).first;
  }
  return it->second;
}

void gmm(at::Tensor a, at::Tensor b, at::Tensor c, at::Tensor batch_sizes, bool trans_a, bool trans_b) {
  // Same checks, in the same order, as csrc/grouped_gemm.cu:476-540.
  TORCH_CHECK(!(trans_a && trans_b), "only one of trans_a / trans_b may be set");
  TORCH_CHECK(batch_sizes.is_cuda() || batch_sizes.is_cpu(), "batch_sizes must be a CPU or CUDA tensor");
  TORCH_CHECK(batch_sizes.dim() == 1, "batch_sizes must be 1-D");
  TORCH_CHECK(batch_sizes.scalar_type() == at::kLong, "batch_sizes must be int64");
  TORCH_CHECK(a.is_cuda(), "a must be a CUDA tensor");
  TORCH_CHECK(a.dim() == 2, "a must be 2-D");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16, "a must be bfloat16");
  TORCH_CHECK(b.is_cuda() && c.is_cuda(), "b and c must be CUDA tensors");
  TORCH_CHECK(b.scalar_type() == at::kBFloat16 && c.scalar_type() == at::kBFloat16,
              "b and c must be bfloat16");
  const int64_t z = batch_sizes.size(0);
  int64_t n = 0;
  if (trans_a) {
    TORCH_CHECK(b.dim() == 2, "b must be 2-D when trans_a is set");
    TORCH_CHECK(c.dim() == 3, "c must be 3-D when trans_a is set");
    TORCH_CHECK(b.size(0) == a.size(0), "a and b must have the same number of rows");
    TORCH_CHECK(c.size(0) == z && c.size(1) == a.size(1) && c.size(2) == b.size(1),
                "c must be [num_experts, a.shape[1], b.shape[1]]");
    n = b.size(1);
  } else {
    TORCH_CHECK(b.dim() == 3, "b must be 3-D");
    TORCH_CHECK(c.dim() == 2, "c must be 2-D");
    const int64_t hidden_in = trans_b ? b.size(2) : b.size(1);
    n = trans_b ? b.size(1) : b.size(2);
    TORCH_CHECK(hidden_in == a.size(1), "contraction dimensions of a and b differ");
    TORCH_CHECK(z == b.size(0), "need one batch size per expert");
    // The reference leaves c's 2-D shape unchecked; a short c would be written
    // out of bounds, so it is checked here.
    TORCH_CHECK(c.size(0) == a.size(0) && c.size(1) == n, "c must be [a.shape[0], hidden_out]");
  }
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && c.is_contiguous(), "a, b and c must be contiguous");
  TORCH_CHECK(a.device() == b.device() && a.device() == c.device(), "a, b and c must be on one device");
  if (batch_sizes.is_cuda()) {
    TORCH_CHECK(batch_sizes.device() == a.device(), "batch_sizes must be on a's device or on the CPU");
    TORCH_CHECK(batch_sizes.is_contiguous(), "batch_sizes must be contiguous");
  } else {
    batch_sizes = batch_sizes.contiguous();
    // The library copies host batch sizes to the device with an asynchronous copy.
    // From pageable memory the data is staged before that call returns; from pinned
    // memory the copy reads the caller's buffer later, on the stream, when the
    // caller may already have changed or freed it.  Take a pageable copy.
    if (batch_sizes.is_pinned()) batch_sizes = batch_sizes.clone();
  }
  TORCH_CHECK(z <= B200GMM_MAX_EXPERTS, b200gmm_strerror(B200GMM_ELIMIT));

  // Integers go into the messages below as std::to_string(...): streaming an int
  // into a TORCH_CHECK message has been seen to crash inside the iostream number
  // facets when libstdc++ versions are mixed; strings are always fine.
  c10::cuda::CUDAGuard guard(a.device());
  size_t ws_bytes = 0;
  int rc = b200gmm_workspace_bytes(static_cast<int>(z), &ws_bytes);
  TORCH_CHECK(rc == 0, "b200gmm_workspace_bytes: ", b200gmm_strerror(rc), " (code ", std::to_string(rc), ")");
  at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)},
                            at::TensorOptions().dtype(at::kByte).device(a.device()));
  at::Tensor status = status_word(a.device());
  rc = b200gmm_run(a.data_ptr(), b.data_ptr(), c.data_ptr(), batch_sizes.data_ptr<int64_t>(),
                   batch_sizes.is_cuda() ? 1 : 0, static_cast<int>(z), a.size(0), a.size(1), n,
                   trans_a ? 1 : 0, trans_b ? 1 : 0, ws.data_ptr(), ws_bytes,
                   reinterpret_cast<uint32_t*>(status.data_ptr<int>()),
                   at::cuda::getCurrentCUDAStream(a.device().index()).stream());
  TORCH_CHECK(rc == 0, "b200gmm_run: ", b200gmm_strerror(rc), " (code ", std::to_string(rc), ")");
}

at::Tensor device_status(int64_t device_index) {
  return status_word(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device_index)));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.def("gmm", &gmm, "Grouped GEMM into caller-provided c (B200, libb200gmm).", py::arg("a"), py::arg("b"),
        py::arg("c"), py::arg("batch_sizes"), py::arg("trans_a"), py::arg("trans_b"));
  m.def("device_status", &device_status, "Per-device status word tensor (int32[1]).",
        py::arg("device_index"));
}
