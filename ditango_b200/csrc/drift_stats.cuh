// Launcher of the drift-metric reduction (drift_stats.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dtb {

constexpr int kDriftTile = 16384;            // elements reduced by one block
constexpr int kDriftScratchHeader = 256;     // ticket counter + padding

inline int64_t drift_blocks(int64_t n) { return n > 0 ? (n + kDriftTile - 1) / kDriftTile : 1; }
inline int64_t drift_scratch_bytes(int64_t n) { return kDriftScratchHeader + drift_blocks(n) * 4 * 8; }

cudaError_t launch_drift_stats(const float* cur, const float* prev, int64_t n, float* accum, unsigned char* scratch,
                               cudaStream_t stream);

}  // namespace dtb
