// The binding a maintainer of the reference would add to route its CUDA branch
// to libot_b200.so: a drop-in for ot::ComputeTransducerLossCuda
// (optimized_transducer/csrc/cuda.cu:402-457 of the reference), called from
// ot::ComputeTransducerLoss (optimized_transducer/csrc/transducer-loss.cc:76-83)
// in place of the original.  It needs nothing but include/ot_b200.h and torch.
//
// This file is an example: it is not part of libot_b200.so.  tests/test_abi.py
// compiles it against the torch headers, so the snippet in INTEGRATION.md (which
// is this function) stays valid C++ against the current header.
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <utility>

#include "ot_b200.h"

namespace ot {

std::pair<torch::Tensor, torch::optional<torch::Tensor>>
ComputeTransducerLossB200(torch::Tensor &logits,  // NOLINT
                          const torch::Tensor &targets,
                          const torch::Tensor &logit_lengths,
                          const torch::Tensor &target_lengths, int32_t blank,
                          bool from_log_softmax, bool one_sym_per_frame) {
  torch::DeviceGuard guard(logits.device());
  const int32_t N = static_cast<int32_t>(logit_lengths.size(0));
  const int32_t V = static_cast<int32_t>(logits.size(1));
  const int32_t max_u = static_cast<int32_t>(targets.size(1));
  const int64_t rows = logits.size(0);
  uint32_t flags = OT_B200_CHECK_INPUTS;  // raise inside the call, as the reference does
  if (from_log_softmax) flags |= OT_B200_FROM_LOG_SOFTMAX;
  if (one_sym_per_frame) flags |= OT_B200_ONE_SYM_PER_FRAME;
  uint64_t bytes = 0;
  TORCH_CHECK(ot_b200_workspace_bytes(N, rows, max_u, flags, &bytes) == OT_B200_OK,
              ot_b200_last_error());
  auto ws = torch::empty({static_cast<int64_t>(bytes)}, logits.options().dtype(torch::kUInt8));
  auto scores = torch::empty({N}, logits.options());
  torch::Tensor grad;  // stays undefined unless logits.requires_grad()
  if (logits.requires_grad())
    grad = from_log_softmax ? torch::empty_like(logits) : logits;  // alias, as cuda.cu:449
  void *stream = c10::cuda::getCurrentCUDAStream().stream();
  const int rc = ot_b200_compute_transducer_loss(
      logits.data_ptr(), grad.defined() ? grad.data_ptr() : nullptr,
      targets.data_ptr<int32_t>(), logit_lengths.data_ptr<int32_t>(),
      target_lengths.data_ptr<int32_t>(), N, rows, V, max_u, blank, flags,
      ws.data_ptr(), bytes, scores.data_ptr(), stream);
  TORCH_CHECK(rc == OT_B200_OK, ot_b200_last_error());
  if (grad.defined()) return {scores, grad};
  return {scores, torch::nullopt};
}

}  // namespace ot
