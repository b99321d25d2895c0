// Selection of split points on (key, index) by most-significant-digit descent: declarations shared by the
// space-filling-curve labels (sfc.cu, where the kernels live) and the KD-tree partition (kdtree.cu).
#pragma once

#include "common.cuh"

namespace dynb {

typedef unsigned __int128 u128;
constexpr int SEL_MAX_SPLITS = 1024;
constexpr int64_t SEL_HIST_BYTES = 4ll << 20;  // per buffer (two buffers)

struct SelSplit {           // one per split point and level parity
    unsigned long long pre_hi, pre_lo;  // C >> (bits not yet decided)
    long long residual;                 // weight still to cover among the atoms that share the prefix
    int dead;                           // its threshold lies beyond the total weight: no atom reaches it
    int pad;
};

__device__ __forceinline__ u128 sel_prefix(const SelSplit& s) { return ((u128)s.pre_hi << 64) | (u128)s.pre_lo; }

// Runs all digit levels on composite numbers C = keys[i] << idx_bits | i (idx_bits = bits of n - 1) and
// returns, through final_out, the device array of nsplit split points whose prefix is then the full
// composite of the split atom (or dead).  thresholds_dev == nullptr: the thresholds of the W-way
// partition (equal counts, or weights_dev); else thresholds_dev[s] = 1 + number of atoms in front of
// split atom s in (key, index) order, non-decreasing in s.  state_ws: 2 * SEL_MAX_SPLITS SelSplit,
// hist_ws: 2 * SEL_HIST_BYTES.  crowded_keys: the keys fall into few values of their leading digit (float
// coordinates): the first level then counts in shared memory first.
int sel_select_splits(const uint64_t* keys_dev, int key_bits, const int64_t* weights_dev, int64_t n, int nsplit, int64_t W,
                      const long long* thresholds_dev, unsigned char* state_ws, unsigned char* hist_ws, int* idx_bits_out,
                      const SelSplit** final_out, bool crowded_keys, cudaStream_t stream);

}  // namespace dynb
