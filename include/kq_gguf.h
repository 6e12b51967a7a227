/*
 * kq_gguf.h - C ABI of libkq: GGUF block-quantized linear kernels for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host runtime binds (ctypes / cgo / a torch extension).  Every entry point
 *   - takes plain device pointers and sizes, never a framework type;
 *   - allocates nothing (except where a comment says otherwise) and never synchronises: work is
 *     enqueued on `stream` (a cudaStream_t passed as void*, NULL = the legacy default stream) of the
 *     CURRENT device, and all scratch memory is the caller's;
 *   - returns 0 on success or a KQ_E* code; kq_last_error() then gives a thread-local message.
 *     (Same convention as the reference's own C-ABI bridges: `int status` + `current_direct_error()`,
 *     vllm_gguf_plugin/native/kernels/current_ggml_direct.cu:32,174.)
 *
 * Each function names the reference interface it replaces (paths inside the kaiLLM source tree).
 *
 * Weight tensors are GGUF wire bytes: uint8 [n, k/blk * block_bytes], rows contiguous, blocks
 * consecutive along k (vllm_gguf_plugin/csrc/gguf/ggml-common.h:20-150).  Supported GGML type ids:
 * 2 (Q4_0), 8 (Q8_0), 10 (Q2_K), 12 (Q4_K), 14 (Q6_K), 21 (IQ3_S) on every path, and 3 (Q4_1), 6 (Q5_0), 7 (Q5_1),
 * 11 (Q3_K), 13 (Q5_K), 20 (IQ4_NL), 23 (IQ4_XS) on the general paths; any other id is KQ_EUNSUPPORTED.
 */
#ifndef KQ_GGUF_H
#define KQ_GGUF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KQ_OK 0
#define KQ_EINVAL 1        /* bad argument (null pointer, negative size, k not a multiple of the block, ...) */
#define KQ_EUNSUPPORTED 2  /* GGML type id or dtype outside the supported set */
#define KQ_ESCRATCH 3      /* scratch buffer missing, misaligned or too small */
#define KQ_ECUDA 4         /* a CUDA runtime call or launch failed; message holds cudaGetErrorString */
#define KQ_ELIMIT 5        /* size beyond a stated maximum of the entry point */

/* element types of activations / outputs */
#define KQ_F32 0
#define KQ_F16 1
#define KQ_BF16 2

/* GGML type ids (gguf-reader/gguf/constants.py:5763-5799) */
#define KQ_TYPE_Q4_0 2
#define KQ_TYPE_Q8_0 8
#define KQ_TYPE_Q2_K 10
#define KQ_TYPE_Q4_K 12
#define KQ_TYPE_Q6_K 14
#define KQ_TYPE_IQ3_S 21
/* the other formats of real mixed-precision checkpoints: served by the general kernels (row-streaming / dp4a GEMV at
 * every m, dequantize), not by the tensor-core paths */
#define KQ_TYPE_Q4_1 3
#define KQ_TYPE_Q5_0 6
#define KQ_TYPE_Q5_1 7
#define KQ_TYPE_Q3_K 11
#define KQ_TYPE_Q5_K 13
#define KQ_TYPE_IQ4_NL 20
#define KQ_TYPE_IQ4_XS 23

/* Thread-local text of the last error returned on this thread ("" if none). */
const char* kq_last_error(void);

/* ABI version of this header (bumped on incompatible change). */
int kq_abi_version(void);

/* Weights per block and bytes per block of a GGML type
 * (gguf-reader/gguf/constants.py:5958 GGML_QUANT_SIZES).  KQ_EUNSUPPORTED for other ids. */
int kq_block_geometry(int type, int* weights_per_block, int* bytes_per_block);

/* Bytes of caller-provided scratch kq_mul_mat_vec_a8 / kq_mul_mat_a8 need for these sizes
 * (quantized activations + split-K partials).  The scratch pointer must be 256-byte aligned.
 * Replaces the `quant_X` allocation in vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:114-115. */
size_t kq_workspace_bytes(int type, int64_t m, int64_t n, int64_t k);

/* q8_1 activation quantizer, reference scratch layout.
 * x: [m, k] row-major with row stride `stride_x` elements, dtype x_dtype.
 * out: m * (kpad/32) blocks of 36 bytes {fp16 d, fp16 sum, int8 q[32]}, kpad = ceil(k/512)*512,
 * positions >= k quantize as zeros.
 * Replaces quantize_row_q8_1_cuda, vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:32-85. */
int kq_quantize_q8_1(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x,
                     void* out_blocks, void* stream);

/* y[m, n] = q8_1(x)[m, k] . W[n, k]^T with the arithmetic of the reference's MMVQ kernels.
 * y has row stride `stride_y` elements and dtype y_dtype (the reference uses x's dtype).
 * Any m >= 1 is accepted; the kernel is chosen inside by m: integer-dot GEMV kernels for m <= 80 (exact
 * integer block dots), the tcgen05 fp16 GEMM above (outputs within rel-L2 1e-3 of the integer arithmetic).
 * Replaces ggml_mul_mat_vec_a8, vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:104-218
 * (kernels: csrc/gguf/mmvq.cuh:2-41, csrc/gguf/vecdotq.cuh). */
int kq_mul_mat_vec_a8(const void* W, int type, int64_t n, int64_t k,
                      const void* x, int x_dtype, int64_t m, int64_t stride_x,
                      void* y, int y_dtype, int64_t stride_y,
                      void* scratch, size_t scratch_bytes, void* stream);

/* Same contract with the arithmetic of the reference's MMQ kernels (Q4_K's min term uses the fp16
 * block sum of the raw activations).  IQ3_S is KQ_EUNSUPPORTED here, as in the reference.
 * Replaces ggml_mul_mat_a8, vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:220-290
 * (kernels: csrc/gguf/mmq.cuh:2-104). */
int kq_mul_mat_a8(const void* W, int type, int64_t n, int64_t k,
                  const void* x, int x_dtype, int64_t m, int64_t stride_x,
                  void* y, int y_dtype, int64_t stride_y,
                  void* scratch, size_t scratch_bytes, void* stream);

/* kq_mul_mat_vec_a8 for hosts that cannot hand over scratch memory.
 * Some embedders of this library own no device allocator at the point of the call: a runtime that has already
 * handed all device memory to its own arena, a plug-in running inside another process's CUDA context under a
 * no-allocation rule, a latency-critical path where cudaMalloc (a device-wide synchronising call) is forbidden.
 * For them this entry point takes no scratch argument: the quantized activations, scale tables and split-K
 * partials live in a device array built into the library image (about 14 MB, held by every GPU that loads the
 * library until the process exits).  Inputs and outputs are still the caller's.  Same arithmetic and same kernels
 * as kq_mul_mat_vec_a8.
 *   Limits: m <= 16, n <= 32768, k <= 32768; anything larger returns KQ_ELIMIT with a message naming the limits.
 *   The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *   current); make that first call outside of any stream capture.  No call allocates or frees device memory.
 *   Every call on a device uses the same array and overwrites what the previous call left there (the counters
 *   that must start at zero are cleared by the call itself), so two calls that may overlap on the GPU - different
 *   streams, or different host threads - race; serialise them on one stream.
 * This entry point has no counterpart in the reference. */
int kq_mul_mat_vec_a8_static(const void* W, int type, int64_t n, int64_t k,
                             const void* x, int x_dtype, int64_t m, int64_t stride_x,
                             void* y, int y_dtype, int64_t stride_y, void* stream);

/* The two halves of the mul_mat entry points, for layers that share one activation (q/k/v, gate/up):
 * kq_prepare_q8 quantizes x into `scratch`; kq_mul_mat_prepared multiplies any number of weight tensors
 * against the activations already held there (mmq != 0 selects the MMQ arithmetic).  n passed to
 * kq_prepare_q8 must be >= every n used with that scratch (it sizes the split-K area; everything the preparation
 * writes sits at offsets that do not depend on n, so weight tensors of different n share one preparation).
 * Tensors of different GGML types may share it too when their blocks have the same number of weights; size the scratch
 * with the largest kq_workspace_bytes over the types (Q4_0 above 16 tokens adds a per-call table).
 * Replace the quantize_row_q8_1_cuda call and the kernel launch inside ggml_mul_mat_vec_a8 /
 * ggml_mul_mat_a8, vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:116-118 and 119-215, 232-287; the
 * reference's production path shares the preparation the same way
 * (vllm_gguf_plugin/quantization/native_fused.py:282-347).
 * flags (also of the fused producers below): 0, or KQ_PREP_WAIT_ARRIVAL when x is a gather buffer that is being filled
 * by kq_mul_mat_prepared_gather calls with wait_in_consumer = 1 (m <= 80): every element is then re-read until it is not
 * the arrival sentinel (all bits set), bounded to about two seconds (status word 40 on give-up). */
#define KQ_PREP_WAIT_ARRIVAL 1
int kq_prepare_q8(int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m, int64_t stride_x,
                  void* scratch, size_t scratch_bytes, int flags, void* stream);
int kq_mul_mat_prepared(const void* W, int type, int64_t n, int64_t k, int64_t m,
                        void* y, int y_dtype, int64_t stride_y, int mmq,
                        void* scratch, size_t scratch_bytes, void* stream);

/* Fused producers for kq_mul_mat_prepared: the activation is computed from its inputs and quantized in ONE launch,
 * bit-identically to running the elementwise / normalising kernel first and kq_prepare_q8 on its output (m <= 80).
 *   kq_prepare_q8_rmsnorm  a = T(T(x * rsqrt(mean(x^2) + eps)) * gamma) with both roundings in the storage type T (the order
 *                          of vLLM's rms_norm kernel); gamma: k values of x_dtype; y_norm (may be NULL): the normalised
 *                          [m, k] tensor, row stride k, for consumers that need it dense
 *   kq_prepare_q8_swiglu   a = T(silu(gate)) * up in T, gate = gate_up[:, 0:k], up = gate_up[:, k:2k] (row stride
 *                          stride_gu >= 2k): vLLM's SiluAndMul on the merged gate/up output, feeding the down projection
 * They take the place of the reference production backend's fused activation producers
 * (vllm_gguf_plugin/native/kernels/kai_prepare_ext.cuh:1-10, quantization/native_fused.py:144-200), with this path's
 * q8_1 arithmetic (gguf_kernel.cu:32-69) instead of that backend's own activation format. */
int kq_prepare_q8_rmsnorm(int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m, int64_t stride_x,
                          const void* gamma, float eps, void* y_norm, void* scratch, size_t scratch_bytes, int flags,
                          void* stream);
int kq_prepare_q8_swiglu(int type, int64_t n, int64_t k, const void* gate_up, int x_dtype, int64_t m, int64_t stride_gu,
                         void* scratch, size_t scratch_bytes, int flags, void* stream);

/* Dense dequantization of `count` weights (count a multiple of the block size) to out_dtype, with
 * the reference kernels' fp16 intermediate roundings.
 * Replaces ggml_dequantize, vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:87-102
 * (kernels: csrc/gguf/dequantize.cuh:3-16,69-121,156-196,232-256,334-353). */
int kq_dequantize(const void* W, int type, int64_t count, void* out, int out_dtype, void* stream);

/* Test hook: exact integer dot products per weight scale group.
 * dots: int32 [m, n, k/G] with G = 16 for Q2_K, Q3_K and Q6_K (one weight scale per 16 weights) and 32 for the others;
 * sums: int32 [m, k/G] = sum of the activation codes of each group (may be NULL).
 * Uses the same scratch as the mul_mat entry points.  No counterpart in the reference (its kernels
 * never materialise the integer dots); exists so the bit-exactness of the integer path can be
 * checked through the ABI. */
int kq_debug_group_dots(const void* W, int type, int64_t n, int64_t k,
                        const void* x, int x_dtype, int64_t m, int64_t stride_x,
                        int32_t* dots, int32_t* sums,
                        void* scratch, size_t scratch_bytes, void* stream);

/* All-gather of the ranks' [M, N/world] output slices by peer stores over NVLink (one kernel, no library
 * collective).  It takes the place of the all-gather that follows a row(N)-sharded linear layer
 * (vLLM's tensor_model_parallel_all_gather behind the column-parallel GGUF layers whose weights
 * quantization/params.py:230-247 shards); the reference itself has no such kernel.
 *   src          this rank's slice (bytes long)
 *   peer_dst     HOST array of `world` device pointers: every rank's gather buffer (world * bytes each), mapped into
 *                this process (e.g. torch symmetric memory); entry `rank` is the local buffer.  The slice lands at
 *                offset rank * bytes of every buffer, so each buffer ends up as [world][M][N/world].
 *   peer_flags   HOST array of `world` device pointers: every rank's flag array, uint32 [slots][8], zero before the
 *                first call
 *   epoch, done  LOCAL device arrays, uint32 [slots], zero before the first call (call counter / CTA counter)
 *   slot         which flag slot this call uses; calls that may be in flight at the same time need different slots
 *   status       LOCAL device int: set non-zero if the bounded wait for a peer's flag ran out (about two seconds; the
 *                kernel then returns early and the local gather buffer is incomplete - treat its contents as undefined)
 * src, the slice size and every peer_dst entry should be 16-byte aligned (16-byte stores); if any of them is not,
 * the copy falls back to single bytes.  Null entries and misaligned flag arrays are KQ_EINVAL.
 * Every rank must make the same sequence of calls per slot.  When the kernel has completed, the local gather buffer
 * holds all ranks' slices.  Alternate two gather buffers per stream if the gathered data is read by later kernels
 * (a peer may write the next call's slice as soon as this rank has published its own next call).
 * world <= 8.  Only plain loads and stores touch peer memory. */
int kq_p2p_allgather(const void* src, size_t bytes, void* const* peer_dst, uint32_t* const* peer_flags,
                     uint32_t* epoch, uint32_t* done, int slot, int rank, int world, int* status, void* stream);

/* The same gather into ROW-MAJOR [M, N] buffers: this rank's slice is [rows][row_bytes] (contiguous) and lands as
 * columns rank * row_bytes .. (rank + 1) * row_bytes of every rank's buffer, whose rows are dst_row_stride bytes apart
 * (>= world * row_bytes).  When the kernel has completed, the local buffer is the layer's full output as the next
 * layer reads it, with no transposing copy.  Everything else as kq_p2p_allgather. */
int kq_p2p_allgather_2d(const void* src, int64_t rows, size_t row_bytes, void* const* peer_dst, size_t dst_row_stride,
                        uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* done, int slot, int rank, int world,
                        int* status, void* stream);

/* A row(N)-sharded linear layer and the all-gather that follows it, as ONE kernel where that is possible: this rank's
 * [n_local, k] slice of the weight matrix times the prepared activations (kq_prepare_q8*), with the outputs stored as
 * columns rank * n_local .. of every rank's row-major [m, stride_y] buffer by plain 16-byte peer stores from the GEMV's
 * own epilogue; the CTA that finishes last raises flag[slot][rank] on every rank and waits (bounded, about two seconds)
 * for theirs, so when the kernel has completed the local buffer is the layer's whole output.  It replaces the pair
 * "ggml_mul_mat_vec_a8 on the rank's shard + tensor_model_parallel_all_gather" of vLLM's column-parallel GGUF layers
 * (shards: vllm_gguf_plugin/quantization/params.py:230-247); the reference has no such kernel.
 *   peer_y       HOST array of `world` device pointers: every rank's output buffer, mapped into this process
 *   stride_y     elements between rows of those buffers (>= world * n_local)
 *   peer_flags, epoch, done, slot, rank, world   as kq_p2p_allgather (the two entries may share flag arrays)
 *   peer_status  LOCAL device int, as `status` of kq_p2p_allgather: set non-zero when the bounded wait for a peer's
 *                flag ran out (16 + rank of the silent peer from the fused kernel, 1 + rank from the gather kernel); the
 *                library never clears it, so one word can watch a whole sequence of calls
 *   wait_in_consumer  0: the hand-shake above.  1: NO hand-shake - the kernel only stores its outputs and returns; every
 *                rank's buffer must hold the arrival sentinel (all bits set) in every element before any rank's call,
 *                and whoever reads the buffer next polls the elements (kq_prepare_q8* with KQ_PREP_WAIT_ARRIVAL, or
 *                kq_wait_arrival before a reader outside the library).  An output that would equal the sentinel (a NaN
 *                with all bits set) is stored as the canonical NaN.  This takes the system-scope fence, the CTA counter
 *                and the flag round trip off the critical path: what remains is the one-way latency of the stores.
 *   reset_buf, reset_bytes  with wait_in_consumer: a LOCAL gather buffer (or NULL) that the producer of this call's
 *                activations has finished reading; the kernel refills it with the sentinel so that its next use starts
 *                from "nothing has arrived" (16-byte aligned and sized).  A buffer may be written again by the peers
 *                only after they have consumed outputs of the call that refilled it - true for a chain of layers where
 *                each call's activations are the previous call's gathered outputs.
 *   fused        out, may be NULL: 1 = one kernel; 0 = two (the usual kernel dispatch into this rank's own columns, then
 *                the gather kernel) - taken for m > 16, for shapes the shared-stage kernel does not cover, for buffers
 *                whose rows are not 16-byte aligned, and with option "no_fused_gather"
 * world == 1 degenerates to kq_mul_mat_prepared. */
int kq_mul_mat_prepared_gather(const void* W, int type, int64_t n_local, int64_t k, int64_t m, int y_dtype, int mmq,
                               void* scratch, size_t scratch_bytes, void* const* peer_y, int64_t stride_y,
                               uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* done, int slot, int rank,
                               int world, int* peer_status, int wait_in_consumer, void* reset_buf, size_t reset_bytes,
                               int* fused, void* stream);

/* Returns (on the stream) when no element of buf holds the arrival sentinel any more: the end of a chain of
 * wait_in_consumer gathers, before something outside the library reads the buffer.  dtype = element type of the buffer
 * (KQ_F32 / KQ_F16 / KQ_BF16); buf 16-byte aligned, bytes a multiple of 16; *status (local device int) becomes 41 when
 * the bounded wait runs out. */
int kq_wait_arrival(const void* buf, size_t bytes, int dtype, int* status, void* stream);

/* Arrival polls that ran out (a peer is gone) set a flag on the GPU that makes every later poll on it give up at once
 * instead of after its own two seconds.  This call copies the flag to *failed (SYNCHRONISES; may be NULL) and, with
 * clear != 0, zeroes it.  0 = no poll has run out since the last clear. */
int kq_arrival_status(int* failed, int clear);

/* Embedding lookup: out[i, :] = the dequantized row row_ids[i] of the [n, k] weight tensor, i < count - the
 * torch.index_select + ggml_dequantize pair of the reference's GGUF embedding (quantization/vocal_embeds.py:38-55) in
 * one kernel, without the gathered copy of the wire rows.  f32_math = 0: arithmetic of kq_dequantize; f32_math = 1, for
 * Q4_K / Q5_K / Q6_K: (d * sc) * q - dmin * m with fp32 products, what gguf-reader computes and what the reference's
 * embedding uses for these three formats (vocal_embeds.py:43-50, triton/dequantize/k_quant/q4_k.py:13-31); other formats
 * ignore the flag.  row_ids: int64 on the device; an index outside [0, n) gives a row of zeros (the reference's
 * index_select traps).  out: [count, k], 16-byte aligned. */
int kq_dequantize_rows(const void* W, int type, int64_t n, int64_t k, const int64_t* row_ids, int64_t count, void* out,
                       int out_dtype, int f32_math, void* stream);

/* ggml_moe_a8_vec (vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:395-530, moe_vec.cuh:4-52): W holds `experts` matrices
 * [n, k] back to back; output row z = token * top_k + j is W[topk_ids[z]] times the q8_1-quantized activations of token
 * z / top_k, with the arithmetic of kq_mul_mat_vec_a8.  x [tokens, k], topk_ids int32 [tokens * top_k] (device), y
 * [tokens * top_k, n].  Rows whose expert id is outside [0, experts) are left as the caller initialised them (the
 * reference reads out of bounds for them).  Scratch: kq_workspace_bytes(type, tokens, n, k).  tokens * top_k <= 65535. */
int kq_moe_a8_vec(const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* x, int x_dtype, int64_t tokens,
                  int64_t stride_x, const int32_t* topk_ids, int top_k, void* y, int y_dtype, int64_t stride_y, void* scratch,
                  size_t scratch_bytes, void* stream);

/* ggml_moe_a8 (gguf_kernel.cu:292-393, moe.cuh:9-128): the (token, expert) pairs sorted by expert in blocks of
 * kq_moe_block_size(type) slots, as vLLM's moe_align_block_size lays them out: block b belongs to expert_ids[b]; slot s
 * holds z = sorted_token_ids[s] (z >= tokens * top_k marks padding) and output row z is W[expert] times the activations
 * of token z / top_k, with the arithmetic of kq_mul_mat_a8.  Blocks that start beyond num_tokens_post_padded[0] and blocks
 * whose expert id is outside [0, experts) (the reference: outside [0, 255]) are skipped; rows nobody writes keep the
 * caller's initialisation (the reference returns zeros).  All three index tensors are int32 on the device;
 * num_sorted = entries of sorted_token_ids (at most 65535 blocks). */
int kq_moe_a8(const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* x, int x_dtype, int64_t tokens,
              int64_t stride_x, const int32_t* sorted_token_ids, int64_t num_sorted, const int32_t* expert_ids,
              const int32_t* num_tokens_post_padded, int top_k, void* y, int y_dtype, int64_t stride_y, void* scratch,
              size_t scratch_bytes, void* stream);

/* ggml_moe_get_block_size (gguf_kernel.cu:532-578): the block size kq_moe_a8 expects of moe_align_block_size (8 for every
 * supported type; the reference's CUDA build answers 4), 0 for a type the library does not know. */
int kq_moe_block_size(int type);

/* Diagnostics: copies the device-side status word of a scratch buffer to the host (SYNCHRONISES with the
 * device; not for the serving path).  0 = every kernel that used the scratch finished normally; non-zero = a
 * bounded wait inside a kernel gave up and the kernel returned early (its outputs are then undefined).
 * The sizes must be the ones the scratch was used with.  No counterpart in the reference. */
int kq_read_status(int type, int64_t m, int64_t n, int64_t k, const void* scratch, size_t scratch_bytes, int* status);

/* The same for the array built into the library that kq_mul_mat_vec_a8_static uses on the current device
 * (SYNCHRONISES; 0 = the kernels of every call so far finished normally).  No counterpart in the reference. */
int kq_read_status_static(int* status);

/* Test hook, host arithmetic only (no GPU work): what the streaming kernels read of a tensor of n rows of rowbytes
 * bytes at address `base` (16-byte aligned).  They stage weight bytes in shared memory with bulk copies of 16-byte
 * units, so they are given only the first `streamed_rows` rows - the largest count whose byte size is a multiple of 16
 * (all n for every even n); the few rows that may remain go to the general kernel, which reads with plain loads.
 * seg_len == 0: whole rows [row_a, row_b); seg_len > 0: bytes [seg_off, seg_off + seg_len) of row row_a.  Returns the
 * bulk-copy range [bulk_start, bulk_start + bulk_bytes) for rows inside the streamed part (0, 0 otherwise).  The
 * kernels and the dispatch call the same functions; a test can assert that nothing outside
 * [base, base + n * rowbytes) is read.  No counterpart in the reference. */
int kq_debug_copy_window(uint64_t base, int64_t n, int64_t rowbytes, int64_t row_a, int64_t row_b, int64_t seg_off,
                         int64_t seg_len, int64_t* streamed_rows, uint64_t* bulk_start, uint64_t* bulk_bytes);

/* Runtime knobs for tests and profiling (process-wide, not thread-safe against concurrent launches):
 *   "gemv_impl"   0 = choose by shape (default), 1 = general dp4a kernel, 3 = row-streaming dp4a kernel,
 *                 4 = the same without the specialised Q4_K / Q6_K consumers, 6 = shared-stage int8-mma kernel,
 *                 7 = register-resident int8-mma kernel, 8 = tensor-memory kernel (tcgen05 kind::i8 MMAs; Q4_K);
 *                 a forced kernel that does not cover the type or shape returns KQ_EUNSUPPORTED
 *   "tc_min_m"    smallest m that the shared-stage int8-mma kernel takes in mode 0 (default 3)
 *   "pdl"         0 = plain launches; p > 0 (default 2) = the quantizer and the streaming kernels are launched
 *                 with programmatic stream serialization and prefetch p ring stages of weights before they
 *                 wait for the previous kernel of the stream
 *   "tile_segments" 1 = the shared-stage kernel fetches row segments even when a stage is contiguous (default 0)
 *   "fuse_q8"     1 (default) = calls of 1-2 tokens on large matrices skip the quantizer launch: the row-streaming
 *                 kernel quantizes the activations itself, bit-identically, while its first weight stages are in
 *                 flight; 2 = wherever that kernel runs (tests); 0 = always launch the quantizer
 *   "kres"        1 (default) = passes of 3..8 tokens use the register-resident kernel where it covers the type and
 *                 shape, 2 = passes of 9..16 tokens too, 0 = never (the shared-stage kernel instead)
 *   "umma"        1 = in mode 0 the tensor-memory kernel takes the passes it covers, from "umma_min_m" tokens on
 *                 (default 0: it is slower than the default kernels today).  The per-unit activation tables it reads
 *                 are only written while it is switched on ("umma" = 1 or "gemv_impl" = 8): set the option BEFORE
 *                 the activations are prepared.  "umma_box" 1 (default) = its weight bytes arrive by tiled TMA copies
 *                 where the rows are 16-byte aligned, 0 = by cp.async
 *   "no_fused_gather" 1 = kq_mul_mat_prepared_gather always runs as two kernels (default 0)
 *   "gemm_min_m"  smallest m that always goes to the tcgen05 GEMM (default 81)
 *   "gemm_small_m" 1 (default) = calls of 17..gemm_min_m-1 tokens go to the GEMM too where one launch beats the
 *                 16-token GEMV passes (Q4_0, Q8_0, Q2_K, Q4_K, Q6_K; k a multiple of 256; from 17 tokens with at least
 *                 120 tiles of 128 rows, from 33 with 60, from 49 with 30; Q4_0 and Q6_K a step later); results then carry
 *                 fp16-operand rounding (rel-L2 about 3e-4 to the
 *                 integer path, inside the 1e-3 contract).  0 = m < gemm_min_m keeps exact integer dots.  Set it
 *                 BEFORE the activations are prepared (kq_prepare_q8* write the GEMM's operands only when wanted)
 *   "row_stage_kb" target size in KB of one shared-memory stage (whole rows) of the Q4_K 1-2-token kernel (default 24)
 *   "tile_two_stage" 1 (default) = the shared-stage GEMV may run on two whole-row stages of >= 32 KB (Q8_0, K = 5120, 9-16
 *                 tokens) instead of splitting K into row segments
 *   "moe_smem"    1 (default) = the MoE ops stage a block's / a pair's activations in shared memory, 0 = one warp per row
 *                 reading them from global memory (bit-identical results)
 *   "gemm_wide"   tile of the GEMM: 0 = 256 rows x 128 tokens, 2 = 128 rows x 256 tokens, 1 (default) = the latter
 *                 whenever more than 128 tokens come or the format's wire bytes are staged through shared memory
 *   "half_fma"    1 = K-quant dequantize contracts fp16 mul+sub into one fma (default), 0 = two roundings
 * Returns KQ_EINVAL for an unknown name. */
int kq_set_option(const char* name, int value);
/* kq_get_option additionally answers "launch_count": kernels launched by the library so far. */
int kq_get_option(const char* name, int* value);

#ifdef __cplusplus
}
#endif
#endif /* KQ_GGUF_H */
