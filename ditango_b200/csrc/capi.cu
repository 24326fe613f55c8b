// C ABI of the library (declared in include/ditango_b200.h): argument checking, TMA tensor-map
// construction and kernel launches.  No entry point allocates device memory.
#include "../../include/ditango_b200.h"

#include "flash_fwd_sm100.cuh"
#include "drift_stats.cuh"
#include "errors.cuh"
#include "merge_states.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// Device status word written by kernels whose bounded waits ran out.
__device__ int g_status_word;

// First code wins, as for codes reported by the kernels themselves.
__global__ void post_status_kernel(int* word, int code) { atomicCAS(word, 0, code); }

struct DeviceInfo {
  bool probed = false;
  int cc_major = 0;
  int sm_count = 0;
  int* status_ptr = nullptr;
};
DeviceInfo g_dev[64];
std::mutex g_mu;

int device_info(DeviceInfo** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(DTB_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceInfo& d = g_dev[dev];
  if (!d.probed) {
    e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "device query failed: %s", cudaGetErrorString(e));
    if (d.cc_major == 10) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_status_word);
      if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      d.status_ptr = static_cast<int*>(p);
    }
    d.probed = true;
  }
  if (d.cc_major != 10) return fail(DTB_ERR_DEVICE, "device %d has compute capability %d.x; sm_100a kernels need 10.x", dev, d.cc_major);
  *out = &d;
  return DTB_OK;
}

}  // namespace

namespace dtb {

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int require_sm100() {
  DeviceInfo* d = nullptr;
  return device_info(&d);
}

}  // namespace dtb

namespace {

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int load_encoder() {
  static std::once_flag once;
  static cudaError_t err = cudaSuccess;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  if (g_encode == nullptr) return fail(DTB_ERR_CUDA, "cuTensorMapEncodeTiled not available: %s", cudaGetErrorString(err));
  return DTB_OK;
}

// 2-D bf16 view [rows, width] with a row pitch of tok_stride elements; boxes of 64 x box_rows elements
// (128 bytes x box_rows rows) written to shared memory with the 128-byte swizzle.
int make_tile_map(CUtensorMap* tm, const void* base, int64_t rows, int64_t width, int64_t tok_stride, int box_rows,
                  const char* what) {
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(tok_stride) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DTB_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, static_cast<int>(r));
  return DTB_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Encoded tensor maps, kept per (base pointer, rows, width, pitch, box rows).  The attention path calls
// with the same few buffers over and over (persistent receive buffers, a layer's q / k / v of a fixed shape),
// so most launches find their three maps here instead of going through the driver's encoder.
struct MapKey {
  const void* base;
  int64_t rows, width, tok_stride;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && width == o.width && tok_stride == o.tok_stride && box_rows == o.box_rows;
  }
};
constexpr int kMapCacheSize = 64;
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool used = false;
};
MapEntry g_maps[kMapCacheSize];
std::mutex g_map_mu;

int cached_tile_map(CUtensorMap* tm, const void* base, int64_t rows, int64_t width, int64_t tok_stride, int box_rows,
                    const char* what) {
  const MapKey key{base, rows, width, tok_stride, box_rows};
  const size_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull + static_cast<size_t>(rows) * 31 +
                   static_cast<size_t>(box_rows);
  const int slot = static_cast<int>((h >> 20) % kMapCacheSize);
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (g_maps[slot].used && g_maps[slot].key == key) {
      *tm = g_maps[slot].map;
      return DTB_OK;
    }
  }
  int rc = make_tile_map(tm, base, rows, width, tok_stride, box_rows, what);
  if (rc != DTB_OK) return rc;
  std::lock_guard<std::mutex> lk(g_map_mu);
  g_maps[slot].key = key;
  g_maps[slot].map = *tm;
  g_maps[slot].used = true;
  return DTB_OK;
}

}  // namespace

#ifdef DTB_FLASH_TIMING
namespace dtb { cudaError_t read_flash_timing(long long* host, int n, int head_dim); }
#endif

extern "C" {

DTB_API int dtb_version(void) { return 100; }

DTB_API const char* dtb_last_error(void) { return g_err; }

DTB_API int dtb_device_supported(void) {
  DeviceInfo* d = nullptr;
  return device_info(&d);
}

DTB_API int dtb_read_status(void* stream) {
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, d->status_ptr, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "status read failed: %s", cudaGetErrorString(e));
  if (host != 0) {
    e = cudaMemsetAsync(d->status_ptr, 0, sizeof(int), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "status clear failed: %s", cudaGetErrorString(e));
    fail(host, "a kernel gave up on a bounded wait (code %d)", host);
  }
  return host;
}

DTB_API int dtb_peek_status_async(int* host_word, void* stream) {
  if (!host_word) return fail(DTB_ERR_ARG, "dtb_peek_status_async: null destination");
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(host_word, d->status_ptr, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "status copy failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int dtb_post_status(int code, void* stream) {
  if (code <= 0) return fail(DTB_ERR_ARG, "dtb_post_status: code must be positive, got %d", code);
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  post_status_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(d->status_ptr, code);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "status write failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int dtb_ipc_export_mem(const void* dev_ptr, void* handle64, int64_t* offset) {
  if (!dev_ptr || !handle64 || !offset) return fail(DTB_ERR_ARG, "dtb_ipc_export_mem: null argument");
  static PFN_cuMemGetAddressRange_v3020 get_range = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      get_range = reinterpret_cast<PFN_cuMemGetAddressRange_v3020>(fn);
  });
  if (get_range == nullptr) return fail(DTB_ERR_CUDA, "dtb_ipc_export_mem: cuMemGetAddressRange not available");
  CUdeviceptr base = 0;
  size_t size = 0;
  CUresult r = get_range(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr));
  if (r != CUDA_SUCCESS) return fail(DTB_ERR_CUDA, "dtb_ipc_export_mem: address range query failed with CUresult %d", static_cast<int>(r));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  static_assert(sizeof(h) == 64, "handle size");
  memcpy(handle64, &h, sizeof(h));
  *offset = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
  return DTB_OK;
}

DTB_API int dtb_ipc_open_mem(const void* handle64, void** base_ptr) {
  if (!handle64 || !base_ptr) return fail(DTB_ERR_ARG, "dtb_ipc_open_mem: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(base_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int dtb_ipc_close_mem(void* base_ptr) {
  if (!base_ptr) return DTB_OK;
  cudaError_t e = cudaIpcCloseMemHandle(base_ptr);
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int dtb_peer_copy_async(void* dst, const void* src, int64_t bytes, void* stream) {
  if (bytes < 0 || (bytes > 0 && (!dst || !src))) return fail(DTB_ERR_ARG, "dtb_peer_copy_async: bad argument");
  if (bytes == 0) return DTB_OK;
  cudaError_t e = cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "peer copy failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

static int flash_fwd_impl(const void* q, const void* k, const void* v,
                          int64_t q_tok_stride, int64_t k_tok_stride, int64_t v_tok_stride,
                          void* out, int out_dtype, int64_t out_tok_stride,
                          float* lse, int lse_layout, int accumulate,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                          int nseg, int seqlen_q, int seqlen_k, int64_t total_q, int64_t total_k,
                          int num_heads, int head_dim, float softmax_scale, int launch_flags, void* stream) {
  if (launch_flags & ~DTB_LAUNCH_OVERLAP_PREVIOUS) return fail(DTB_ERR_ARG, "dtb_flash_fwd: unknown launch flag 0x%x", launch_flags);
  if (!q || !k || !v || !out || !lse) return fail(DTB_ERR_ARG, "dtb_flash_fwd: null tensor pointer");
  if (head_dim != 64 && head_dim != 128) return fail(DTB_ERR_ARG, "dtb_flash_fwd: head_dim %d not in {64, 128}", head_dim);
  if (num_heads < 1 || num_heads > 65535) return fail(DTB_ERR_ARG, "dtb_flash_fwd: num_heads %d out of range", num_heads);
  if (nseg < 1 || nseg > 65535) return fail(DTB_ERR_ARG, "dtb_flash_fwd: nseg %d out of range", nseg);
  if (seqlen_q < 0 || seqlen_k < 0 || total_q < 0 || total_k < 0) return fail(DTB_ERR_ARG, "dtb_flash_fwd: negative length");
  if (total_q >= (1ll << 31) || total_k >= (1ll << 31)) return fail(DTB_ERR_ARG, "dtb_flash_fwd: more than 2^31 tokens");
  if ((cu_seqlens_q == nullptr) != (cu_seqlens_k == nullptr)) return fail(DTB_ERR_ARG, "dtb_flash_fwd: cu_seqlens_q and cu_seqlens_k must both be given or both be null");
  if (cu_seqlens_q == nullptr && (static_cast<int64_t>(nseg) * seqlen_q > total_q || static_cast<int64_t>(nseg) * seqlen_k > total_k))
    return fail(DTB_ERR_ARG, "dtb_flash_fwd: nseg*seqlen exceeds total tokens");
  const int64_t width = static_cast<int64_t>(num_heads) * head_dim;
  if (q_tok_stride < width || k_tok_stride < width || v_tok_stride < width || out_tok_stride < width)
    return fail(DTB_ERR_ARG, "dtb_flash_fwd: token stride smaller than num_heads*head_dim");
  if ((q_tok_stride | k_tok_stride | v_tok_stride | out_tok_stride) & 7) return fail(DTB_ERR_ARG, "dtb_flash_fwd: token strides must be multiples of 8 elements");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return fail(DTB_ERR_ARG, "dtb_flash_fwd: tensor pointers must be 16-byte aligned");
  if (out_dtype != DTB_F32 && out_dtype != DTB_BF16) return fail(DTB_ERR_ARG, "dtb_flash_fwd: bad out_dtype %d", out_dtype);
  if (lse_layout != DTB_LSE_BHS && lse_layout != DTB_LSE_BSH) return fail(DTB_ERR_ARG, "dtb_flash_fwd: bad lse_layout %d", lse_layout);
  if (accumulate && out_dtype != DTB_F32) return fail(DTB_ERR_ARG, "dtb_flash_fwd: accumulate needs an fp32 state");
  if (!(softmax_scale > 0.f)) return fail(DTB_ERR_ARG, "dtb_flash_fwd: softmax_scale must be positive");
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  if (seqlen_q == 0 || total_q == 0) return DTB_OK;
  rc = load_encoder();
  if (rc != DTB_OK) return rc;

  CUtensorMap tq, tk, tv;
  // A tensor map needs at least one row; an empty key chunk never issues a load.
  const int64_t rows_k = total_k > 0 ? total_k : 1;
  const int kv_rows = dtb::flash_kv_box_rows(head_dim);
  if ((rc = cached_tile_map(&tq, q, total_q, width, q_tok_stride, 128, "q")) != DTB_OK) return rc;
  if ((rc = cached_tile_map(&tk, k, rows_k, width, k_tok_stride, kv_rows, "k")) != DTB_OK) return rc;
  if ((rc = cached_tile_map(&tv, v, rows_k, width, v_tok_stride, kv_rows, "v")) != DTB_OK) return rc;

  dtb::FlashParams p;
  p.out = out;
  p.lse = lse;
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.status = d->status_ptr;
  p.out_tok_stride = out_tok_stride;
  p.total_q = total_q;
  p.nseg = nseg;
  p.seqlen_q = seqlen_q;
  p.seqlen_k = seqlen_k;
  p.num_heads = num_heads;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.out_dtype = out_dtype;
  p.lse_layout = lse_layout;
  p.accumulate = accumulate ? 1 : 0;
  p.overlap_previous = (launch_flags & DTB_LAUNCH_OVERLAP_PREVIOUS) ? 1 : 0;
  cudaError_t e = (head_dim == 64) ? dtb::launch_flash<64>(tq, tk, tv, p, static_cast<cudaStream_t>(stream))
                                   : dtb::launch_flash<128>(tq, tk, tv, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "dtb_flash_fwd launch failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int dtb_flash_fwd(const void* q, const void* k, const void* v,
                  int64_t q_tok_stride, int64_t k_tok_stride, int64_t v_tok_stride,
                  void* out, int out_dtype, int64_t out_tok_stride,
                  float* lse, int lse_layout, int accumulate,
                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                  int nseg, int seqlen_q, int seqlen_k, int64_t total_q, int64_t total_k,
                  int num_heads, int head_dim, float softmax_scale, void* stream) {
  return flash_fwd_impl(q, k, v, q_tok_stride, k_tok_stride, v_tok_stride, out, out_dtype, out_tok_stride, lse, lse_layout,
                        accumulate, cu_seqlens_q, cu_seqlens_k, nseg, seqlen_q, seqlen_k, total_q, total_k, num_heads,
                        head_dim, softmax_scale, 0, stream);
}

DTB_API int dtb_flash_fwd_ex(const void* q, const void* k, const void* v,
                     int64_t q_tok_stride, int64_t k_tok_stride, int64_t v_tok_stride,
                     void* out, int out_dtype, int64_t out_tok_stride,
                     float* lse, int lse_layout, int accumulate,
                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                     int nseg, int seqlen_q, int seqlen_k, int64_t total_q, int64_t total_k,
                     int num_heads, int head_dim, float softmax_scale, int launch_flags, void* stream) {
  return flash_fwd_impl(q, k, v, q_tok_stride, k_tok_stride, v_tok_stride, out, out_dtype, out_tok_stride, lse, lse_layout,
                        accumulate, cu_seqlens_q, cu_seqlens_k, nseg, seqlen_q, seqlen_k, total_q, total_k, num_heads,
                        head_dim, softmax_scale, launch_flags, stream);
}

DTB_API int dtb_merge_states(int nstates, const void* const* outs, const int* out_dtypes,
                     const float* const* lses, const int* lse_layouts,
                     float* out, float* lse_out, int lse_out_layout, void* out_bf16,
                     int batch, int seq, int num_heads, int head_dim, void* stream) {
  if (nstates < 1 || nstates > DTB_MERGE_MAX_STATES) return fail(DTB_ERR_ARG, "dtb_merge_states: nstates %d not in [1, %d]", nstates, DTB_MERGE_MAX_STATES);
  if (head_dim != 64 && head_dim != 128) return fail(DTB_ERR_ARG, "dtb_merge_states: head_dim %d not in {64, 128}", head_dim);
  if (!outs || !out_dtypes || !lses || !lse_layouts) return fail(DTB_ERR_ARG, "dtb_merge_states: null argument");
  if (!out && !out_bf16) return fail(DTB_ERR_ARG, "dtb_merge_states: neither an fp32 nor a bf16 result buffer was given");
  if (batch < 0 || seq < 0 || num_heads < 1) return fail(DTB_ERR_ARG, "dtb_merge_states: bad shape");
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  dtb::MergeParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < nstates; ++i) {
    if (!outs[i] || !lses[i]) return fail(DTB_ERR_ARG, "dtb_merge_states: state %d has a null pointer", i);
    if (!aligned16(outs[i])) return fail(DTB_ERR_ARG, "dtb_merge_states: state %d is not 16-byte aligned", i);
    if (out_dtypes[i] != DTB_F32 && out_dtypes[i] != DTB_BF16) return fail(DTB_ERR_ARG, "dtb_merge_states: bad dtype for state %d", i);
    if (lse_layouts[i] != DTB_LSE_BHS && lse_layouts[i] != DTB_LSE_BSH) return fail(DTB_ERR_ARG, "dtb_merge_states: bad lse layout for state %d", i);
    if (i > 0 && ((out && outs[i] == out) || (lse_out && lses[i] == lse_out))) return fail(DTB_ERR_ARG, "dtb_merge_states: the result may alias state 0 only");
    p.outs[i] = outs[i];
    p.lse[i] = lses[i];
    p.out_dtype[i] = out_dtypes[i];
    p.lse_layout[i] = lse_layouts[i];
  }
  if (out && outs[0] == out && out_dtypes[0] != DTB_F32) return fail(DTB_ERR_ARG, "dtb_merge_states: in-place merge needs an fp32 state 0");
  if (lse_out && lses[0] == lse_out && lse_layouts[0] != lse_out_layout) return fail(DTB_ERR_ARG, "dtb_merge_states: in-place lse needs matching layouts");
  if ((out && !aligned16(out)) || (out_bf16 && !aligned16(out_bf16))) return fail(DTB_ERR_ARG, "dtb_merge_states: result not 16-byte aligned");
  p.out = out;
  p.lse_out = lse_out;
  p.out_bf16 = static_cast<uint16_t*>(out_bf16);
  p.rows = static_cast<int64_t>(batch) * seq * num_heads;
  p.lse_out_layout = lse_out_layout;
  p.nstates = nstates;
  p.H = num_heads;
  p.S = seq;
  if (p.rows == 0) return DTB_OK;
  cudaError_t e = dtb::launch_merge(p, head_dim, d->sm_count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "dtb_merge_states launch failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int dtb_copy_chunks(int npairs, const void* const* srcs, void* const* dsts, int64_t chunk_bytes,
                    int64_t n0, int64_t n1, int64_t n2,
                    int64_t ss0, int64_t ss1, int64_t ss2,
                    int64_t ds0, int64_t ds1, int64_t ds2, void* stream) {
  if (npairs < 1 || npairs > 4) return fail(DTB_ERR_ARG, "dtb_copy_chunks: npairs %d not in [1, 4]", npairs);
  if (!srcs || !dsts) return fail(DTB_ERR_ARG, "dtb_copy_chunks: null argument");
  if (chunk_bytes <= 0 || (chunk_bytes & 15)) return fail(DTB_ERR_ARG, "dtb_copy_chunks: chunk_bytes must be a positive multiple of 16");
  if ((ss0 | ss1 | ss2 | ds0 | ds1 | ds2) & 15) return fail(DTB_ERR_ARG, "dtb_copy_chunks: strides must be multiples of 16 bytes");
  if (n0 < 0 || n1 < 0 || n2 < 0) return fail(DTB_ERR_ARG, "dtb_copy_chunks: negative extent");
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  dtb::CopyParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < npairs; ++i) {
    if (!srcs[i] || !dsts[i] || !aligned16(srcs[i]) || !aligned16(dsts[i])) return fail(DTB_ERR_ARG, "dtb_copy_chunks: pair %d null or misaligned", i);
    p.src[i] = srcs[i];
    p.dst[i] = dsts[i];
  }
  p.chunk_bytes = chunk_bytes;
  p.n0 = n0; p.n1 = n1; p.n2 = n2;
  p.ss0 = ss0; p.ss1 = ss1; p.ss2 = ss2;
  p.ds0 = ds0; p.ds1 = ds1; p.ds2 = ds2;
  if (n0 * n1 * n2 == 0) return DTB_OK;
  cudaError_t e = dtb::launch_copy_chunks(p, npairs, d->sm_count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "dtb_copy_chunks launch failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

DTB_API int64_t dtb_drift_scratch_bytes(int64_t n) { return dtb::drift_scratch_bytes(n < 0 ? 0 : n); }

DTB_API int dtb_drift_accumulate(const float* cur, const float* prev, int64_t n, float* accum,
                                 void* scratch, int64_t scratch_bytes, void* stream) {
  if (n < 0) return fail(DTB_ERR_ARG, "dtb_drift_accumulate: negative length");
  if (!accum || !scratch || (n > 0 && (!cur || !prev))) return fail(DTB_ERR_ARG, "dtb_drift_accumulate: null pointer");
  if (reinterpret_cast<uintptr_t>(scratch) & 255) return fail(DTB_ERR_ARG, "dtb_drift_accumulate: scratch must be 256-byte aligned");
  if (scratch_bytes < dtb::drift_scratch_bytes(n))
    return fail(DTB_ERR_ARG, "dtb_drift_accumulate: scratch of %lld bytes is smaller than the %lld needed for n = %lld",
                static_cast<long long>(scratch_bytes), static_cast<long long>(dtb::drift_scratch_bytes(n)), static_cast<long long>(n));
  if (dtb::drift_blocks(n) >= (1ll << 31)) return fail(DTB_ERR_ARG, "dtb_drift_accumulate: n too large");
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != DTB_OK) return rc;
  cudaError_t e = dtb::launch_drift_stats(cur, prev, n, accum, static_cast<unsigned char*>(scratch), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(DTB_ERR_CUDA, "dtb_drift_accumulate launch failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

#ifdef DTB_FLASH_TIMING
DTB_API int dtb_debug_flash_timing(long long* host, int n, int head_dim) {
  return dtb::read_flash_timing(host, n, head_dim) == cudaSuccess ? 0 : DTB_ERR_CUDA;
}
#endif

}  // extern "C"
