// Exposes the intermediate stages of the reference's CPU implementation.
//
// TEST INFRASTRUCTURE ONLY.  The reference keeps its stage functions
// (log-prob gather, alpha, beta) file-static in optimized_transducer/csrc/cpu.cc,
// so this translation unit textually includes that file, unmodified and from
// where the reference tree lies (the include path is given by build_ref.py),
// and binds the statics for the parity tests.  No reference source is copied.
#include "optimized_transducer/csrc/cpu.cc"  // NOLINT(build/include)
#include "torch/extension.h"

namespace {

std::pair<torch::Tensor, torch::Tensor> Alpha(const torch::Tensor &lp,
                                              const torch::Tensor &T,
                                              const torch::Tensor &U,
                                              bool one_sym_per_frame) {
  return one_sym_per_frame ? ot::ComputeAlphaOneSymPerFrame(lp, T, U)
                           : ot::ComputeAlpha(lp, T, U);
}

std::pair<torch::Tensor, torch::Tensor> Beta(const torch::Tensor &lp,
                                             const torch::Tensor &T,
                                             const torch::Tensor &U,
                                             bool one_sym_per_frame) {
  return one_sym_per_frame ? ot::ComputeBetaOneSymPerFrame(lp, T, U)
                           : ot::ComputeBeta(lp, T, U);
}

torch::Tensor LogProbs(const torch::Tensor &logits, const torch::Tensor &targets,
                       const torch::Tensor &T, const torch::Tensor &U,
                       int32_t blank, bool from_log_softmax) {
  if (from_log_softmax)
    return ot::ComputeLogProbsForLogSoftmax(logits, targets, T, U, blank);
  torch::Tensor den = logits.logsumexp(1, false);  // as cpu.cc:770
  return ot::ComputeLogProbs(logits, den, targets, T, U, blank);
}

}  // namespace

PYBIND11_MODULE(_ot_ref_stages, m) {
  m.doc() = "stage-level access to the reference CPU implementation";
  m.def("log_probs", &LogProbs, py::arg("logits"), py::arg("targets"),
        py::arg("logit_lengths"), py::arg("target_lengths"), py::arg("blank"),
        py::arg("from_log_softmax"));
  m.def("alpha", &Alpha, py::arg("log_probs"), py::arg("logit_lengths"),
        py::arg("target_lengths"), py::arg("one_sym_per_frame"));
  m.def("beta", &Beta, py::arg("log_probs"), py::arg("logit_lengths"),
        py::arg("target_lengths"), py::arg("one_sym_per_frame"));
}
