// Host-side dataset index construction (pybind11 + numpy, no device code).
//
//   build_sample_idx        GPT: (document position, token offset) of every training sample
//   build_blending_indices  which dataset, and which sample of it, each blended sample comes from
//   build_mapping           sentence-span samples (start, end, target length) for masked-LM data
//   build_blocks_mapping    (start, end, document, block id) blocks for retrieval-style data
//
// Same Python-visible behaviour as the reference's helper module
// (eth/runtime/megatron/data/helpers.cpp:36-96, 99-185, 203-467, 469-710).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cstdint>
#include <iostream>
#include <random>
#include <stdexcept>
#include <vector>

namespace py = pybind11;

namespace {

constexpr int kLongSentence = 512;

// Deterministic Fisher-Yates over rows of `width` values.
template <typename T>
void shuffle_rows(std::vector<T>& v, int width, uint64_t seed) {
  const int64_t n = static_cast<int64_t>(v.size()) / width;
  std::mt19937_64 gen(seed);
  for (int64_t i = n - 1; i > 0; --i) {
    const int64_t j = static_cast<int64_t>(gen() % static_cast<uint64_t>(i + 1));
    for (int k = 0; k < width; ++k) std::swap(v[i * width + k], v[j * width + k]);
  }
}

template <typename T>
py::array to_array(std::vector<T>&& data, int64_t rows, int width) {
  auto* heap = new std::vector<T>(std::move(data));
  py::capsule owner(heap, [](void* p) { delete reinterpret_cast<std::vector<T>*>(p); });
  return py::array(py::dtype::of<T>(), {rows, static_cast<int64_t>(width)},
                   {static_cast<int64_t>(width * sizeof(T)), static_cast<int64_t>(sizeof(T))}, heap->data(), owner);
}

int target_length(int short_ratio, int max_length, std::mt19937& gen) {
  // with probability 1/short_ratio pick a shorter target in [2, max_length]
  if (short_ratio == 0) return max_length;
  const auto r = gen();
  if (r % static_cast<uint32_t>(short_ratio) == 0) return 2 + static_cast<int>(r % static_cast<uint32_t>(max_length - 1));
  return max_length;
}

}  // namespace

void build_blending_indices(py::array_t<uint8_t>& dataset_index, py::array_t<int64_t>& dataset_sample_index,
                            const py::array_t<double>& weights, const int32_t num_datasets, const int64_t size,
                            const bool verbose) {
  auto di = dataset_index.mutable_unchecked<1>();
  auto dsi = dataset_sample_index.mutable_unchecked<1>();
  auto w = weights.unchecked<1>();
  std::vector<int64_t> taken(num_datasets, 0);
  for (int64_t s = 0; s < size; ++s) {
    const double pos = std::max(static_cast<double>(s), 1.0);
    int64_t pick = 0;
    double worst = w[0] * pos - static_cast<double>(taken[0]);
    for (int64_t d = 1; d < num_datasets; ++d) {
      const double err = w[d] * pos - static_cast<double>(taken[d]);
      if (err > worst) { worst = err; pick = d; }
    }
    di[s] = static_cast<uint8_t>(pick);
    dsi[s] = taken[pick]++;
  }
  if (verbose) {
    std::cout << " > sample ratios:" << std::endl;
    for (int64_t d = 0; d < num_datasets; ++d)
      std::cout << "   dataset " << d << ", input: " << w[d] << ", achieved: "
                << static_cast<double>(taken[d]) / static_cast<double>(size) << std::endl;
  }
}

py::array build_sample_idx(const py::array_t<int32_t>& sizes_, const py::array_t<int32_t>& doc_idx_,
                           const int32_t seq_length, const int32_t num_epochs, const int64_t tokens_per_epoch) {
  if (seq_length <= 1 || num_epochs <= 0 || tokens_per_epoch <= 1) throw std::invalid_argument("bad sample index sizes");
  auto sizes = sizes_.unchecked<1>();
  auto doc_idx = doc_idx_.unchecked<1>();
  const int64_t num_samples = (static_cast<int64_t>(num_epochs) * tokens_per_epoch - 1) / seq_length;
  std::vector<int32_t> out(2 * (num_samples + 1));
  int64_t pos = 0;       // position inside doc_idx
  int32_t offset = 0;    // token offset inside the current document
  out[0] = 0; out[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int32_t need = seq_length + 1;   // consecutive samples share one token
    while (need != 0) {
      const int32_t left = sizes[doc_idx[pos]] - offset;
      need -= left;
      if (need <= 0) {
        offset += need + left - 1;
        need = 0;
      } else {
        ++pos;
        offset = 0;
      }
    }
    out[2 * s] = static_cast<int32_t>(pos);
    out[2 * s + 1] = offset;
  }
  return to_array<int32_t>(std::move(out), num_samples + 1, 2);
}

py::array build_mapping(const py::array_t<int64_t>& docs_, const py::array_t<int>& sizes_, const int num_epochs,
                        const uint64_t max_num_samples, const int max_seq_length, const double short_seq_prob,
                        const int seed, const bool verbose, const int32_t min_num_sent) {
  if (num_epochs <= 0 || max_seq_length <= 1 || short_seq_prob < 0.0 || short_seq_prob > 1.0)
    throw std::invalid_argument("bad mapping arguments");
  auto docs = docs_.unchecked<1>();
  auto sizes = sizes_.unchecked<1>();
  const int short_ratio = short_seq_prob > 0 ? static_cast<int>(1.0 / short_seq_prob + 0.5) : 0;
  std::vector<uint64_t> out;
  std::mt19937 gen(static_cast<uint32_t>(seed));
  uint64_t emitted = 0;
  for (int epoch = 0; epoch < num_epochs && emitted < max_num_samples; ++epoch) {
    for (int64_t d = 0; d + 1 < docs.shape(0) && emitted < max_num_samples; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      if (last - first < min_num_sent) continue;
      bool has_long = false;
      for (int64_t s = first; s < last; ++s) has_long |= sizes[s] > kLongSentence;
      if (has_long) continue;
      int64_t start = first;
      int len = 0, count = 0;
      int target = target_length(short_ratio, max_seq_length, gen);
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++count;
        const int64_t remaining = last - s - 1;
        if ((len >= target && remaining >= min_num_sent && count >= min_num_sent) || remaining == 0) {
          if (count >= min_num_sent || remaining == 0) {
            if (count >= min_num_sent) {
              out.push_back(static_cast<uint64_t>(start));
              out.push_back(static_cast<uint64_t>(s + 1));
              out.push_back(static_cast<uint64_t>(target));
              ++emitted;
            }
            start = s + 1;
            len = 0;
            count = 0;
            target = target_length(short_ratio, max_seq_length, gen);
          }
        }
      }
    }
  }
  if (verbose) std::cout << "    built " << emitted << " sentence-span samples" << std::endl;
  shuffle_rows(out, 3, static_cast<uint64_t>(seed) + 1);
  const int64_t rows = static_cast<int64_t>(out.size() / 3);
  return to_array<uint64_t>(std::move(out), rows, 3);
}

py::array build_blocks_mapping(const py::array_t<int64_t>& docs_, const py::array_t<int>& sizes_,
                               const py::array_t<int>& titles_sizes_, const int num_epochs,
                               const uint64_t max_num_samples, const int max_seq_length, const int seed,
                               const bool verbose, const bool use_one_sent_blocks) {
  if (num_epochs <= 0 || max_seq_length <= 1) throw std::invalid_argument("bad block mapping arguments");
  auto docs = docs_.unchecked<1>();
  auto sizes = sizes_.unchecked<1>();
  auto titles = titles_sizes_.unchecked<1>();
  const int min_sent = use_one_sent_blocks ? 1 : 2;
  std::vector<uint64_t> out;
  uint64_t emitted = 0;
  for (int epoch = 0; epoch < num_epochs && emitted < max_num_samples; ++epoch) {
    uint64_t block_id = 0;
    for (int64_t d = 0; d + 1 < docs.shape(0) && emitted < max_num_samples; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      const int budget = max_seq_length - titles[d];
      if (last - first < min_sent || budget <= 0) continue;
      bool has_long = false;
      for (int64_t s = first; s < last; ++s) has_long |= sizes[s] > kLongSentence;
      if (has_long) continue;
      int64_t start = first;
      int len = 0, count = 0;
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++count;
        const int64_t remaining = last - s - 1;
        if ((len >= budget && (remaining >= min_sent || remaining == 0) && count >= min_sent) || remaining == 0) {
          if (count >= min_sent) {
            out.push_back(static_cast<uint64_t>(start));
            out.push_back(static_cast<uint64_t>(s + 1));
            out.push_back(static_cast<uint64_t>(d));
            out.push_back(block_id++);
            ++emitted;
          }
          start = s + 1;
          len = 0;
          count = 0;
        }
      }
    }
  }
  if (verbose) std::cout << "    built " << emitted << " blocks" << std::endl;
  shuffle_rows(out, 4, static_cast<uint64_t>(seed) + 1);
  const int64_t rows = static_cast<int64_t>(out.size() / 4);
  return to_array<uint64_t>(std::move(out), rows, 4);
}

PYBIND11_MODULE(_data_helpers, m) {
  m.def("build_mapping", &build_mapping);
  m.def("build_blocks_mapping", &build_blocks_mapping);
  m.def("build_sample_idx", &build_sample_idx);
  m.def("build_blending_indices", &build_blending_indices);
}
