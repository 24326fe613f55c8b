// Parameters and launcher of the partial-attention forward kernels (flash_fwd_sm100.cu picks between
// flash_fwd_row.cu and flash_fwd_pair.cu by head dimension).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dtb {

struct FlashParams {
  void* out;               // fp32 or bf16, token stride out_tok_stride, head h at h*D
  float* lse;              // fp32, natural log
  const int32_t* cu_q;     // device cumulative offsets (packed batch) or nullptr (dense batch)
  const int32_t* cu_k;
  int* status;             // device status word (0 = ok)
  int64_t out_tok_stride;  // elements
  int64_t total_q;         // tokens behind q
  int nseg;                // sequences (dense: batch size)
  int seqlen_q;            // dense: exact; packed: upper bound per segment
  int seqlen_k;
  int num_heads;
  float scale_log2;        // softmax_scale * log2(e)
  int out_dtype;           // 0 fp32, 1 bf16
  int lse_layout;          // 0 [B,H,S] (packed: [H,T]), 1 [B,S,H]
  int accumulate;          // merge into the state already in (out, lse)
  int overlap_previous;    // host only: launch with programmatic stream serialization (see launch_flash)
};

// With p.overlap_previous the launch may begin while the previous launch on `stream` is finishing (its CTAs fill
// the SMs that kernel's last wave leaves idle).  The kernels read q, k, v, cu_seqlens before they wait for that
// kernel and touch (out, lse) only after it has completed, so this is allowed exactly when the last kernel or copy
// queued on the stream is another launch_flash whose results this launch does not read as q, k, v or cu_seqlens
// (event waits and records in between do not matter).
template <int D>
cudaError_t launch_flash(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                         const FlashParams& p, cudaStream_t stream);

// Rows of one K / V tile: the tensor maps of k and v must be encoded with boxes of 64 x this many elements
// (q always uses 64 x 128).
int flash_kv_box_rows(int head_dim);

}  // namespace dtb
