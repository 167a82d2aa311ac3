// CPU index builders for the memory-mapped GPT dataset stack (same three entry
// points and numpy contracts as lm_engine/data/megatron/utils/helpers.cpp:17-233
// of the reference, so cached index files are interchangeable):
//   build_blending_indices  - interleave samples of several datasets so that the
//                             running mix tracks the requested weights as closely as possible
//   build_sample_idx_int32 / _int64 - (document index, offset) of the start of every
//                             training sample when documents are concatenated and cut into
//                             windows of seq_length + 1 tokens that overlap by one token
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cstdint>
#include <iostream>
#include <stdexcept>
#include <vector>

namespace py = pybind11;

namespace b200 {

namespace {

void build_blending_indices(py::array_t<int16_t>& dataset_index, py::array_t<int64_t>& dataset_sample_index,
                            const py::array_t<double>& weights, const int32_t num_datasets, const int64_t size,
                            const bool verbose) {
  auto which = dataset_index.mutable_unchecked<1>();
  auto where = dataset_sample_index.mutable_unchecked<1>();
  auto w = weights.unchecked<1>();
  if (verbose) std::cout << "> building indices for blended datasets ..." << std::endl;

  std::vector<int64_t> drawn(num_datasets, 0);
  for (int64_t i = 0; i < size; ++i) {
    // The dataset that lags its target share the most gets the next sample.
    const double denom = static_cast<double>(std::max<int64_t>(i, 1));
    int64_t pick = 0;
    double worst = w[0] * denom - static_cast<double>(drawn[0]);
    for (int32_t d = 1; d < num_datasets; ++d) {
      const double lag = w[d] * denom - static_cast<double>(drawn[d]);
      if (lag > worst) {
        worst = lag;
        pick = d;
      }
    }
    which[i] = static_cast<int16_t>(pick);
    where[i] = drawn[pick];
    drawn[pick] += 1;
  }

  if (verbose) {
    std::cout << " > sample ratios:" << std::endl;
    for (int32_t d = 0; d < num_datasets; ++d) {
      const double achieved = static_cast<double>(drawn[d]) / static_cast<double>(size);
      std::cout << "   dataset " << d << ", input: " << w[d] << ", achieved: " << achieved << std::endl;
    }
  }
}

template <typename OutT>
py::array build_sample_idx(const py::array_t<int32_t>& sizes_, const py::array_t<OutT>& doc_idx_,
                           const int32_t seq_length, const int32_t num_epochs, const int64_t tokens_per_epoch) {
  if (seq_length <= 1 || num_epochs <= 0 || tokens_per_epoch <= 1) {
    throw std::invalid_argument("build_sample_idx: seq_length > 1, num_epochs > 0 and tokens_per_epoch > 1 required");
  }
  auto sizes = sizes_.unchecked<1>();
  auto doc_idx = doc_idx_.template unchecked<1>();

  const int64_t num_samples = (static_cast<int64_t>(num_epochs) * tokens_per_epoch - 1) / seq_length;
  // The result owns its storage through a capsule whose deleter matches the allocation type.
  auto* table = new std::vector<OutT>(static_cast<size_t>(2 * (num_samples + 1)));
  OutT* out = table->data();

  int64_t doc_cursor = 0;  // position in doc_idx
  OutT offset = 0;         // token offset inside the current document
  out[0] = static_cast<OutT>(doc_cursor);
  out[1] = offset;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int64_t need = static_cast<int64_t>(seq_length) + 1;
    while (need != 0) {
      const int64_t doc_len = static_cast<int64_t>(sizes[doc_idx[doc_cursor]]) - static_cast<int64_t>(offset);
      need -= doc_len;
      if (need <= 0) {
        // The window ends inside this document; the next window re-reads its last token.
        offset = static_cast<OutT>(static_cast<int64_t>(offset) + need + doc_len - 1);
        need = 0;
      } else {
        ++doc_cursor;
        offset = 0;
      }
    }
    out[2 * s] = static_cast<OutT>(doc_cursor);
    out[2 * s + 1] = offset;
  }

  py::capsule owner(table, [](void* p) { delete reinterpret_cast<std::vector<OutT>*>(p); });
  const auto stride = static_cast<py::ssize_t>(sizeof(OutT));
  return py::array(py::dtype::of<OutT>(), {num_samples + 1, static_cast<int64_t>(2)}, {2 * stride, stride}, out, owner);
}

}  // namespace

void register_data_helpers(py::module_& m) {
  m.def("build_blending_indices", &build_blending_indices);
  m.def("build_sample_idx_int32", &build_sample_idx<int32_t>);
  m.def("build_sample_idx_int64", &build_sample_idx<int64_t>);
}

}  // namespace b200
