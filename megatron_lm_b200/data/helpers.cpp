// CPU index builders for the dataset pipeline (C ABI, loaded with ctypes).
//
// Same jobs as the reference's pybind11 module megatron/core/datasets/helpers.cpp
// (build_sample_idx :142, build_blending_indices :75, build_exhaustive_blending_indices :21,
// build_mapping :266/:526, build_blocks_mapping :564/:805), written as flat loops over caller-owned
// numpy buffers: the caller sizes the outputs (a first call with out == nullptr returns the count).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <random>
#include <vector>

extern "C" {

// Number of samples a packed GPT dataset yields.
int64_t mlb_num_samples(int64_t num_epochs, int64_t tokens_per_epoch, int32_t seq_length, int32_t add_extra_token,
                        int32_t drop_last_partial) {
  const int64_t total = num_epochs * tokens_per_epoch - add_extra_token;
  if (drop_last_partial) return total / seq_length;
  return (total + seq_length - 1) / seq_length;
}

// sample_idx[(n+1) * 2]: position in document_idx and token offset where each sample starts.
// A sample is seq_length (+1 if add_extra_token) tokens and may span documents.
// idx64 selects the width of document_idx (int32 or int64).  Returns 0, or -1 on inconsistent input.
int mlb_build_sample_idx(const int32_t* sizes, const void* document_idx, int32_t idx64, int64_t document_idx_len,
                         int32_t seq_length, int64_t num_samples, int32_t add_extra_token,
                         int32_t drop_last_partial, int64_t* sample_idx) {
  auto doc_at = [&](int64_t i) -> int64_t {
    return idx64 ? static_cast<const int64_t*>(document_idx)[i] : static_cast<const int32_t*>(document_idx)[i];
  };
  int64_t pos = 0;        // index into document_idx
  int64_t offset = 0;     // token offset inside that document
  sample_idx[0] = 0;
  sample_idx[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int64_t need = static_cast<int64_t>(seq_length) + add_extra_token;
    while (need > 0) {
      if (pos >= document_idx_len) return -1;
      const int64_t avail = static_cast<int64_t>(sizes[doc_at(pos)]) - offset;
      if (avail >= need) {
        // the sample ends inside this document; the next one re-reads the last token when an
        // extra (label) token is part of every sample
        offset += need - add_extra_token;
        need = 0;
      } else {
        need -= avail;
        if (pos == document_idx_len - 1) {
          // ran out of documents: only legal for the final partial sample
          if (drop_last_partial || s != num_samples) return -1;
          offset = static_cast<int64_t>(sizes[doc_at(pos)]) - add_extra_token;
          need = 0;
        } else {
          ++pos;
          offset = 0;
        }
      }
    }
    sample_idx[2 * s] = pos;
    sample_idx[2 * s + 1] = offset;
  }
  return 0;
}

// Greedy blend: sample i goes to the dataset whose realised share lags its weight the most.
void mlb_build_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index, const double* weights,
                                int32_t num_datasets, int64_t size) {
  std::vector<int64_t> taken(num_datasets, 0);
  for (int64_t i = 0; i < size; ++i) {
    const double denom = static_cast<double>(std::max<int64_t>(i, 1));
    int32_t best = 0;
    double best_err = weights[0] * denom - static_cast<double>(taken[0]);
    for (int32_t d = 1; d < num_datasets; ++d) {
      const double err = weights[d] * denom - static_cast<double>(taken[d]);
      if (err > best_err) { best_err = err; best = d; }
    }
    dataset_index[i] = static_cast<int16_t>(best);
    dataset_sample_index[i] = taken[best];
    ++taken[best];
  }
}

// Blend that uses every sample of every dataset exactly once (sizes[d] samples from dataset d),
// interleaved in proportion to the sizes.
void mlb_build_exhaustive_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index,
                                           const int64_t* sizes, int32_t num_datasets) {
  int64_t total = 0;
  for (int32_t d = 0; d < num_datasets; ++d) total += sizes[d];
  std::vector<double> w(num_datasets);
  for (int32_t d = 0; d < num_datasets; ++d) w[d] = total ? static_cast<double>(sizes[d]) / total : 0.0;
  std::vector<int64_t> taken(num_datasets, 0);
  for (int64_t i = 0; i < total; ++i) {
    const double denom = static_cast<double>(std::max<int64_t>(i, 1));
    int32_t best = -1;
    double best_err = 0.0;
    for (int32_t d = 0; d < num_datasets; ++d) {
      if (taken[d] >= sizes[d]) continue;
      const double err = w[d] * denom - static_cast<double>(taken[d]);
      if (best < 0 || err > best_err) { best_err = err; best = d; }
    }
    dataset_index[i] = static_cast<int16_t>(best);
    dataset_sample_index[i] = taken[best];
    ++taken[best];
  }
}

// Sentence-pair sample map for BERT-style datasets.  docs[d]..docs[d+1] is the sentence range of
// document d, sizes[] the sentence lengths.  Each output row is (first sentence, one past the last
// sentence, target sequence length).  Documents with fewer than min_num_sent sentences or with a
// sentence longer than 512 tokens are skipped.  With probability short_seq_prob the target length
// is drawn uniformly from [2, max_seq_length].  Pass out == nullptr to count rows.  Rows are
// shuffled with a Mersenne twister seeded by seed + 1.
int64_t mlb_build_mapping(const int64_t* docs, int64_t num_docs, const int32_t* sizes, int32_t num_epochs,
                          int64_t max_num_samples, int32_t max_seq_length, double short_seq_prob, int32_t seed,
                          int32_t min_num_sent, int64_t* out) {
  const int32_t kLongSentence = 512;
  int64_t count = 0;
  std::mt19937 gen(static_cast<uint32_t>(seed));
  auto target_len = [&]() -> int32_t {
    if (short_seq_prob <= 0.0) return max_seq_length;
    const uint32_t r = gen();
    const double u = (r % 1000003u) / 1000003.0;
    if (u < short_seq_prob) return 2 + static_cast<int32_t>(gen() % static_cast<uint32_t>(max_seq_length - 1));
    return max_seq_length;
  };
  for (int32_t epoch = 0; epoch < num_epochs && count < max_num_samples; ++epoch) {
    for (int64_t d = 0; d < num_docs && count < max_num_samples; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      if (last - first < min_num_sent) continue;
      bool too_long = false;
      for (int64_t s = first; s < last; ++s) if (sizes[s] > kLongSentence) { too_long = true; break; }
      if (too_long) continue;
      int64_t start = first;
      int32_t len = 0, nsent = 0;
      int32_t target = target_len();
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++nsent;
        const int64_t remain = last - s - 1;
        if ((len >= target && remain >= min_num_sent && nsent >= min_num_sent) || remain == 0) {
          if (nsent >= min_num_sent || remain == 0) {
            if (out) { out[3 * count] = start; out[3 * count + 1] = s + 1; out[3 * count + 2] = target; }
            ++count;
            if (count >= max_num_samples) break;
          }
          start = s + 1;
          len = 0;
          nsent = 0;
          target = target_len();
        }
      }
    }
  }
  if (out && count > 1) {
    std::mt19937_64 sh(static_cast<uint64_t>(seed) + 1);
    for (int64_t i = count - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(sh() % static_cast<uint64_t>(i + 1));
      for (int k = 0; k < 3; ++k) std::swap(out[3 * i + k], out[3 * j + k]);
    }
  }
  return count;
}

// Block map for inverse-cloze / retrieval datasets: rows of (first sentence, one past last, document,
// block id); a block packs whole sentences up to max_seq_length minus the title length.
int64_t mlb_build_blocks_mapping(const int64_t* docs, int64_t num_docs, const int32_t* sizes,
                                 const int32_t* title_sizes, int32_t num_epochs, int64_t max_num_samples,
                                 int32_t max_seq_length, int32_t seed, int32_t use_one_sent_blocks, int64_t* out) {
  const int32_t kLongSentence = 512;
  const int32_t min_sent = use_one_sent_blocks ? 1 : 2;
  int64_t count = 0;
  for (int32_t epoch = 0; epoch < num_epochs && count < max_num_samples; ++epoch) {
    int64_t block_id = 0;
    for (int64_t d = 0; d < num_docs && count < max_num_samples; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      if (last - first < min_sent) continue;
      bool too_long = false;
      for (int64_t s = first; s < last; ++s) if (sizes[s] > kLongSentence) { too_long = true; break; }
      if (too_long) continue;
      const int32_t budget = max_seq_length - title_sizes[d];
      int64_t start = first;
      int32_t len = 0, nsent = 0;
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++nsent;
        const int64_t remain = last - s - 1;
        if ((len >= budget && remain >= min_sent && nsent >= min_sent) || remain == 0) {
          if (out) {
            out[4 * count] = start; out[4 * count + 1] = s + 1; out[4 * count + 2] = d; out[4 * count + 3] = block_id;
          }
          ++count;
          ++block_id;
          if (count >= max_num_samples) break;
          start = s + 1;
          len = 0;
          nsent = 0;
        }
      }
    }
  }
  if (out && count > 1) {
    std::mt19937_64 sh(static_cast<uint64_t>(seed) + 1);
    for (int64_t i = count - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(sh() % static_cast<uint64_t>(i + 1));
      for (int k = 0; k < 4; ++k) std::swap(out[4 * i + k], out[4 * j + k]);
    }
  }
  return count;
}

}  // extern "C"
