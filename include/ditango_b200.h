/*
 * ditango_b200 -- C ABI of the sm_100a kernels behind DiTango's sequence-parallel attention path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*), launches asynchronously on that stream and returns an int
 * status: 0 = launched; negative = rejected argument (nothing was launched, text in
 * dtb_last_error()).  Pointers are borrowed: the caller keeps the memory alive until the
 * stream has passed the call.  Nothing here allocates device memory.  The calling thread's
 * current CUDA device must be the one that owns the pointers.
 *
 * Citations name the reference call site each entry point replaces (paths relative to the
 * reference project root).
 */
#ifndef DITANGO_B200_H_
#define DITANGO_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DTB_API __attribute__((visibility("default")))
#else
#define DTB_API
#endif

#define DTB_OK 0
#define DTB_ERR_ARG (-1)      /* unsupported shape / null pointer / misaligned pointer          */
#define DTB_ERR_CUDA (-2)     /* a CUDA runtime or driver call failed (launch, tensor map, ...) */
#define DTB_ERR_DEVICE (-3)   /* current device is not compute capability 10.x                  */

/* element types of partial-state outputs */
#define DTB_F32 0
#define DTB_BF16 1

/* layouts of a log-sum-exp tensor that belongs to tokens [B,S] x heads H
 * (packed inputs: B = 1, S = total tokens) */
#define DTB_LSE_BHS 0         /* [B, H, S]  -- what flash_attn returns                         */
#define DTB_LSE_BSH 1         /* [B, S, H]  -- the merged state's [B,S,H,1]                    */

#define DTB_MERGE_MAX_STATES 16

DTB_API int dtb_version(void);

/* Text of the last rejected call on this host thread ("" if none). */
DTB_API const char* dtb_last_error(void);

/* 0 if the current device can run these kernels (compute capability 10.x), else DTB_ERR_DEVICE. */
DTB_API int dtb_device_supported(void);

/*
 * Device-side status word.  Kernels that wait on hardware barriers bound every wait; a wait that
 * runs out records a non-zero code and the kernel returns without storing results.
 * dtb_read_status synchronises `stream`, returns the word (0 = all kernels completed normally)
 * and clears it.
 */
DTB_API int dtb_read_status(void* stream);

/*
 * The word is sticky: once a wait has run out, every later launch of these kernels sees a non-zero
 * word in its prologue and returns without doing its work, so that nothing runs on a pipeline whose
 * state is unknown -- and nothing is stored, so results from then on are not valid although every
 * launch call returns 0.  A caller must therefore look at the word, either with dtb_read_status at a
 * point where a synchronisation is acceptable, or without blocking: dtb_peek_status_async queues a
 * copy of the word into *host_word (pinned host memory, owned by the caller) on `stream`; the value
 * is valid once work queued before the call on that stream has completed (an event recorded behind
 * it has fired).  The reference has no counterpart; its failure mode for a stuck transfer is a hung
 * process (core/group_coordinate.py:664-668 waits without a limit).
 *
 * dtb_post_status lets the host set the word (code > 0), ordered on `stream`: a watchdog that learnt
 * on the host that a peer rank is gone uses it to make kernels in flight give up their waits (they
 * poll the word) and to stop later launches, instead of letting each wait run to its limit.
 */
DTB_API int dtb_peek_status_async(int* host_word, void* stream);
DTB_API int dtb_post_status(int code, void* stream);

/*
 * Copy-engine KV transport between the GPUs of one node.  Replaces the NCCL send / receive pairs behind
 * GroupCoordinator.p2p_isend / p2p_irecv / p2p_commit (core/group_coordinate.py:643-668) as used by
 * async_ring_p2p_commit (core/attention.py:37-62): the owner of a KV chunk writes it straight into a
 * receive buffer of the consumer with one asynchronous device-to-device copy, which a copy engine
 * executes -- no SM is taken from the attention kernel.
 *
 *  dtb_ipc_export_mem   consumer side: the 64-byte CUDA IPC handle of the allocation that contains
 *                       dev_ptr, and dev_ptr's byte offset inside it (the caller ships both to the peer).
 *  dtb_ipc_open_mem     owner side: maps the peer's allocation into this process for the CURRENT device
 *                       (peer access is enabled on demand) and returns its base address; add the offset.
 *                       Map a handle once and keep it; close it with dtb_ipc_close_mem at shutdown.
 *  dtb_peer_copy_async  one asynchronous copy of `bytes` from src to dst on `stream` (either may be
 *                       peer-mapped memory).  One call per copy.
 * Ordering between the two processes is the caller's job (interprocess CUDA events plus a host-side
 * handshake; see ditango_b200/core/peer_transport.py).  These calls allocate nothing.
 */
DTB_API int dtb_ipc_export_mem(const void* dev_ptr, void* handle64, int64_t* offset);
DTB_API int dtb_ipc_open_mem(const void* handle64, void** base_ptr);
DTB_API int dtb_ipc_close_mem(void* base_ptr);
DTB_API int dtb_peer_copy_async(void* dst, const void* src, int64_t bytes, void* stream);

/*
 * Partial attention state of a query chunk against ONE key/value chunk (non-causal, no dropout):
 *     S = scale * Q K^T,  lse = logsumexp_k S,  out = softmax_k(S) V
 * Replaces flash_attn_func(q, k, v, dropout_p=0, return_attn_probs=True) at
 * core/attention.py:137-143 and :185-191, flash_attn_varlen_func at :314-324 and :366-376, and
 * _flash_attn_varlen_forward at baseline/ulysses.py:99-113.
 *
 *  q, k, v        bf16.  Token t, head h, channel c of q is q[t*q_tok_stride + h*head_dim + c]
 *                 (likewise k, v): [B,S,H,D] or packed [T,H,D] tensors, or slices of wider rows.
 *                 Base pointers 16-byte aligned, strides multiples of 8 elements.
 *  out            out_dtype DTB_F32 or DTB_BF16, same indexing with out_tok_stride.
 *  lse            fp32, natural-log units, layout lse_layout over (nseg or 1, tokens, heads).
 *  accumulate     0: write this chunk's state to (out, lse).
 *                 1: merge this chunk's state INTO the state already held in (out, lse)
 *                    (out must be DTB_F32) -- the update_out_and_lse step of utils.py:24-84 done
 *                    in the kernel's epilogue.  A row whose lse holds -inf is treated as empty.
 *  cu_seqlens_q/k NULL: dense batch -- nseg sequences of exactly seqlen_q query and seqlen_k key
 *                 tokens each, stored back to back.  Otherwise device int32[nseg+1] cumulative
 *                 offsets of a packed batch; seqlen_q / seqlen_k are then upper bounds on a
 *                 segment's length.  Segment i of q attends segment i of k.  Rows of a segment
 *                 with no keys get out = 0, lse = -inf.
 *  total_q/k      number of tokens addressable behind q / k,v (rows of the 2-D view).
 *  head_dim       64 or 128.
 */
DTB_API int dtb_flash_fwd(const void* q, const void* k, const void* v,
                  int64_t q_tok_stride, int64_t k_tok_stride, int64_t v_tok_stride,
                  void* out, int out_dtype, int64_t out_tok_stride,
                  float* lse, int lse_layout, int accumulate,
                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                  int nseg, int seqlen_q, int seqlen_k, int64_t total_q, int64_t total_k,
                  int num_heads, int head_dim, float softmax_scale, void* stream);

/*
 * dtb_flash_fwd with launch flags.  The reference walks the chunks of a ring block with one attention call
 * per chunk (core/attention.py:160-196); on the device these are back-to-back launches whose grids do not
 * divide evenly over the SMs, so every launch ends with a partly filled wave.
 *
 *  DTB_LAUNCH_OVERLAP_PREVIOUS   this launch may start while the operation queued just before it on `stream`
 *      is finishing: its CTAs take the SMs that launch's last wave leaves idle (programmatic dependent
 *      launch).  The kernel reads q, k, v and cu_seqlens at once, and waits for the previous launch to
 *      complete before it reads or writes (out, lse) -- so accumulating into the state the previous launch
 *      wrote is fine.  Contract: the last kernel or copy queued on `stream` before this call must be another
 *      dtb_flash_fwd / dtb_flash_fwd_ex launch, and this call's q, k, v, cu_seqlens must not be produced by
 *      it.  Event waits and event records in between are fine (they write no memory and do not stop the
 *      overlap).  After any other kernel or a copy pass 0: what the operation just before wrote is only
 *      guaranteed visible to a launch without the flag.
 */
#define DTB_LAUNCH_OVERLAP_PREVIOUS 1
DTB_API int dtb_flash_fwd_ex(const void* q, const void* k, const void* v,
                     int64_t q_tok_stride, int64_t k_tok_stride, int64_t v_tok_stride,
                     void* out, int out_dtype, int64_t out_tok_stride,
                     float* lse, int lse_layout, int accumulate,
                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                     int nseg, int seqlen_q, int seqlen_k, int64_t total_q, int64_t total_k,
                     int num_heads, int head_dim, float softmax_scale, int launch_flags, void* stream);

/*
 * N-way merge of partial softmax states in one pass over HBM:
 *     lse_out = log sum_i exp(lse_i),   out = sum_i exp(lse_i - lse_out) * out_i
 * Replaces the chains of update_out_and_lse (utils.py:24-84) at core/attention.py:110-116, :144,
 * :193-196, :213 and proCache._merge_blocks (core/cache.py:28-46).
 *
 *  outs[i]       state i's values, [rows_bs, H, D] contiguous, dtype out_dtypes[i]
 *  lses[i]       state i's fp32 lse over the same tokens, layout lse_layouts[i]
 *  out / lse_out fp32 results (lse_out may be NULL); `out` and `lse_out` may alias input 0 only.
 *  out_bf16      optional copy of the result in bf16 (NULL to skip): the cast the reference's
 *                callers apply right after the call (executor/cogvideox/attention_processor.py:80).
 *                When it is given, `out` may be NULL and the fp32 result is not written at all.
 *  batch, seq    tokens are [batch, seq]; they matter for DTB_LSE_BHS indexing only.
 *  States whose lse is -inf on a row contribute nothing; a row empty in all states gets
 *  out = 0, lse = -inf.
 */
DTB_API int dtb_merge_states(int nstates, const void* const* outs, const int* out_dtypes,
                     const float* const* lses, const int* lse_layouts,
                     float* out, float* lse_out, int lse_out_layout, void* out_bf16,
                     int batch, int seq, int num_heads, int head_dim, void* stream);

/*
 * Strided copy of contiguous chunks: for every (i0,i1,i2) in [n0,n1,n2) copies chunk_bytes from
 * src + i0*ss0 + i1*ss1 + i2*ss2 to dst + i0*ds0 + i1*ds1 + i2*ds2 (strides in bytes), for each of
 * `npairs` (src, dst) pairs in one launch.  chunk_bytes, strides and pointers are multiples of 16.
 * Used for the head<->sequence re-layouts around the Ulysses all-to-all, replacing the
 * tensor_split + contiguous + cat copies of GroupCoordinator.all_to_all
 * (core/group_coordinate.py:281-286).
 */
DTB_API int dtb_copy_chunks(int npairs, const void* const* srcs, void* const* dsts, int64_t chunk_bytes,
                    int64_t n0, int64_t n1, int64_t n2,
                    int64_t ss0, int64_t ss1, int64_t ss2,
                    int64_t ds0, int64_t ds1, int64_t ds2, void* stream);

/*
 * Drift metric of the redundancy-profiling pass, accumulated on the device:
 *     *accum += mean|cur - prev| / (mean|prev| + 1e-8)      over positions where neither is NaN
 * (mean|cur| instead when mean|prev| < 1e-6; +inf when no position is valid).  Replaces rel_l1
 * (utils.py:202-267) as called from RedundancyMap.record_out_redundancy
 * (core/redundancy_map.py:174-197), which reads three means back to the host per layer and step.
 *
 *  cur, prev     fp32 [n] on the device
 *  accum         one fp32 on the device (for example an element of the [steps, layers] map)
 *  scratch       device memory of at least dtb_drift_scratch_bytes(n) bytes, 256-byte aligned, whose
 *                first 4 bytes are zero before the first call; the call leaves them zero, so one
 *                buffer serves any number of calls that do not overlap on the device.
 */
DTB_API int64_t dtb_drift_scratch_bytes(int64_t n);
DTB_API int dtb_drift_accumulate(const float* cur, const float* prev, int64_t n, float* accum,
                                 void* scratch, int64_t scratch_bytes, void* stream);

/*
 * dtb_drift_accumulate for callers that cannot supply (or allocate) scratch memory.  It has no
 * counterpart in the reference.  Same result as dtb_drift_accumulate; the partial sums go into a
 * 1 MiB array built into the library's device image, which every GPU that loads the library holds
 * until the process exits.  No cudaMalloc / cudaFree or allocating library routine is called.
 *
 *  - n is limited to dtb_drift_noalloc_max_elements() (536,739,840); larger inputs are rejected
 *    with DTB_ERR_ARG and a message naming the limit.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and remembers it; make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's contents; the
 *    entry point clears the one word that must start at zero.  Two calls that overlap on the GPU
 *    (different streams, or different host threads) race on it: serialise them.
 */
DTB_API int64_t dtb_drift_noalloc_max_elements(void);
DTB_API int dtb_drift_accumulate_noalloc(const float* cur, const float* prev, int64_t n, float* accum, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DITANGO_B200_H_ */
