// Parameters and launchers of the state-merge and chunk-copy kernels (merge_states.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dtb {

constexpr int kMergeMaxStates = 16;

struct MergeParams {
  const void* outs[kMergeMaxStates];    // [rows, D] fp32 or bf16
  const float* lse[kMergeMaxStates];
  int out_dtype[kMergeMaxStates];       // 0 fp32, 1 bf16
  int lse_layout[kMergeMaxStates];      // 0 [B,H,S], 1 [B,S,H]
  float* out;                           // [rows, D] fp32
  float* lse_out;                       // may be null
  uint16_t* out_bf16;                   // may be null
  int64_t rows;                         // B*S*H
  int lse_out_layout;
  int nstates;
  int H;
  int S;
};

struct CopyParams {
  const void* src[4];
  void* dst[4];
  int64_t chunk_bytes;
  int64_t n0, n1, n2;
  int64_t ss0, ss1, ss2;
  int64_t ds0, ds1, ds2;
};

cudaError_t launch_merge(const MergeParams& p, int head_dim, int sm_count, cudaStream_t stream);
cudaError_t launch_copy_chunks(const CopyParams& p, int npairs, int sm_count, cudaStream_t stream);

}  // namespace dtb
