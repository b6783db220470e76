// Host-side index builders for the token datasets (C ABI, loaded through ctypes).
//
//  neox_build_sample_idx   : walk the (shuffled, epoch-repeated) document order and cut it into
//                            samples of seq_length + 1 tokens; emits [num_samples + 1, 2] rows of
//                            (index into doc_idx, token offset inside that document).
//  neox_build_blending_indices : interleave several datasets so that after every prefix the realised
//                            mixture is as close as possible to the requested weights (greedy:
//                            pick the dataset with the largest deficit).
//  neox_build_shuffle_idx  : Fisher-Yates permutation with a 64-bit Mersenne twister.
//
// These replace the pybind11 module megatron/data/helpers.cpp:34-259 of the reference; results of the
// first two are defined by the algorithm, so they match it exactly.
#include <cstdint>
#include <cstring>
#include <random>
#include <vector>
#include <algorithm>

extern "C" {

// sizes: int32[num_docs_total]; doc_idx: int32[doc_idx_len]; out: int64[(num_samples+1)*2]
// returns the number of rows written (num_samples + 1) or -1 on inconsistent input.
long long neox_build_sample_idx(const int32_t* sizes, const int32_t* doc_idx, long long doc_idx_len,
                                int32_t seq_length, int32_t num_epochs, long long tokens_per_epoch,
                                long long* out, long long out_rows) {
    const long long num_samples = (static_cast<long long>(num_epochs) * tokens_per_epoch - 1) / seq_length;
    if (out_rows < num_samples + 1) return -1;
    long long sample = 0, di = 0;
    int32_t offset = 0;
    out[0] = di;
    out[1] = offset;
    ++sample;
    while (sample <= num_samples) {
        int32_t remaining = seq_length + 1;
        while (remaining != 0) {
            if (di >= doc_idx_len) return -1;
            const int32_t doc_len = sizes[doc_idx[di]] - offset;
            remaining -= doc_len;
            if (remaining <= 0) {
                // the sample ends inside this document; the next one starts on its last token
                offset += remaining + doc_len - 1;
                remaining = 0;
            } else {
                ++di;
                offset = 0;
            }
        }
        out[2 * sample] = di;
        out[2 * sample + 1] = offset;
        ++sample;
    }
    return num_samples + 1;
}

void neox_build_blending_indices(uint8_t* dataset_index, long long* dataset_sample_index, const double* weights,
                                 int32_t num_datasets, long long size) {
    std::vector<long long> taken(num_datasets, 0);
    for (long long i = 0; i < size; ++i) {
        const double denom = std::max(static_cast<double>(i), 1.0);
        int best = 0;
        double best_err = weights[0] * denom - static_cast<double>(taken[0]);
        for (int d = 1; d < num_datasets; ++d) {
            const double err = weights[d] * denom - static_cast<double>(taken[d]);
            if (err > best_err) {
                best_err = err;
                best = d;
            }
        }
        dataset_index[i] = static_cast<uint8_t>(best);
        dataset_sample_index[i] = taken[best];
        ++taken[best];
    }
}

void neox_build_shuffle_idx(long long* out, long long n, unsigned long long seed) {
    for (long long i = 0; i < n; ++i) out[i] = i;
    std::mt19937_64 gen(seed);
    for (long long i = n - 1; i > 0; --i) {
        std::uniform_int_distribution<long long> pick(0, i);
        std::swap(out[i], out[pick(gen)]);
    }
}

}  // extern "C"
