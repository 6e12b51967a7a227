// Shared definitions of libkq: GGUF block geometry, error plumbing, q8 scratch layout and the
// per-format decode of one 32-weight sub-block into dp4a/MMA-ready int8 words.
//
// Block layouts follow vllm_gguf_plugin/csrc/gguf/ggml-common.h:20-150 of the reference tree.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kq_gguf.h"

namespace kq {

// ------------------------------------------------------------------ host side plumbing
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
#define KQ_CUDA_TRY(expr)                                  \
  do {                                                     \
    cudaError_t _e = (expr);                               \
    if (_e != cudaSuccess) return ::kq::cuda_fail(_e, #expr); \
  } while (0)

// One-time set-up that belongs to a (function, device) pair, e.g. cudaFuncSetAttribute: a flag per device ordinal.
// Setting an attribute twice is harmless, so two threads racing on the first call need no lock.
struct DeviceOnce {
  bool set[64] = {};
  int dev = -1;
  bool first_time() {
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { dev = -1; return true; }
    return !set[dev];
  }
  void done() { if (dev >= 0) set[dev] = true; }
};
int sm_count();   // multiprocessors of the CURRENT device (cached per device ordinal)

struct Options {
  int gemv_impl;       // 0 auto, 1 general dp4a, 3 row-streaming dp4a, 4 same without the specialised consumers,
                       // 6 shared-stage mma (token-major tiles)
  int tc_min_m;        // auto mode: smallest token count that goes to the tensor-core consumers
  int gemm_min_m;      // smallest token count that goes to the tcgen05 GEMM
  int pdl;             // 0: plain launches; p > 0: programmatic dependent launch, p ring stages prefetched before
                       // the kernel waits for its predecessor
  int half_fma;        // 1: fp16 mul+sub contracted in K-quant dequantize
  long long launches;  // kernels launched by this library so far (host-side count)
  int tile_segments;   // 1: the tile GEMV fetches row segments even when its K slice is the whole row
  int fuse_q8;         // 1: calls of 1-2 tokens quantize the activations inside the row-streaming kernel (no quantizer launch)
  int kres;            // 1: passes of 3..8 tokens use the register-resident kernel where it covers the type and shape;
                       // 2: passes of 9..16 tokens as well (slower than the shared-stage kernel today); 0: never
  int umma;            // 1: the tensor-memory decode kernel takes the passes it covers (auto mode)
  int umma_min_m;      // ... from this many tokens on
  int umma_box;        // 1: its weight bytes arrive by tiled TMA copies where the rows are 16-byte aligned (else cp.async)
  int no_fused_gather; // 1: kq_mul_mat_prepared_gather always runs as two kernels (GEMV, then the gather kernel)
  int gemm_wide;       // tcgen05 GEMM tile: 0 = 256 rows x 128 tokens, 2 = 128 rows x 256 tokens, 1 = the latter when m > 128
                       // or the format's wire bytes are staged through shared memory (where it is faster at every m)
  int row_stage_kb;    // Q4_K row-pair GEMV (1-2 tokens): target size of one ring stage (whole rows) in KB
  int tile_two_stage;  // 1: the shared-stage GEMV may run on two whole-row stages of >= 32 KB instead of splitting K
  int moe_smem;        // 1: the MoE ops stage a block's / a pair's activations in shared memory (0: the one-warp-per-row kernel)
  int gemm_small_m;    // 1: calls of 17..gemm_min_m-1 tokens also go to the tcgen05 GEMM where it beats the 16-token
                       // GEMV passes (staged formats, enough 128-row tiles to fill the GPU)
};
Options& options();

// ------------------------------------------------------------------ formats
template <int QT> struct Fmt;
template <> struct Fmt<KQ_TYPE_Q4_0> { static constexpr int BLK = 32, BYTES = 18, GROUP = 32; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_Q8_0> { static constexpr int BLK = 32, BYTES = 34, GROUP = 32; static constexpr bool HAS_MIN = false; };
template <> struct Fmt<KQ_TYPE_Q2_K> { static constexpr int BLK = 256, BYTES = 84, GROUP = 16; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_Q4_K> { static constexpr int BLK = 256, BYTES = 144, GROUP = 32; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_Q6_K> { static constexpr int BLK = 256, BYTES = 210, GROUP = 16; static constexpr bool HAS_MIN = false; };
template <> struct Fmt<KQ_TYPE_IQ3_S> { static constexpr int BLK = 256, BYTES = 110, GROUP = 32; static constexpr bool HAS_MIN = false; };
template <> struct Fmt<KQ_TYPE_Q4_1> { static constexpr int BLK = 32, BYTES = 20, GROUP = 32; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_Q5_0> { static constexpr int BLK = 32, BYTES = 22, GROUP = 32; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_Q5_1> { static constexpr int BLK = 32, BYTES = 24, GROUP = 32; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_Q3_K> { static constexpr int BLK = 256, BYTES = 110, GROUP = 16; static constexpr bool HAS_MIN = false; };
template <> struct Fmt<KQ_TYPE_Q5_K> { static constexpr int BLK = 256, BYTES = 176, GROUP = 32; static constexpr bool HAS_MIN = true; };
template <> struct Fmt<KQ_TYPE_IQ4_NL> { static constexpr int BLK = 32, BYTES = 18, GROUP = 32; static constexpr bool HAS_MIN = false; };
template <> struct Fmt<KQ_TYPE_IQ4_XS> { static constexpr int BLK = 256, BYTES = 136, GROUP = 32; static constexpr bool HAS_MIN = false; };
// Q4_1 / Q5_1: the reference forms d * d8 and m * s8 in fp16 (__hmul2) before using them in fp32
// (vecdotq.cuh:71-92, 131-160); wb carries -m, z is the raw fp16 block sum
template <int QT> struct HalfProd { static constexpr bool value = QT == KQ_TYPE_Q4_1 || QT == KQ_TYPE_Q5_1; };
// min term from the fp16 RAW block sum (true) or from d8 * (sum of the codes) (false), per format and flavour:
// Q4_0 always raw (vecdotq.cuh:46-66); Q4_K / Q5_K raw in the MMQ flavour only (:353-379, :405-445); Q5_0 raw in the
// MMVQ flavour (:94-126) and exact in MMQ (its tile loader subtracts 16 from the codes)
template <int QT, bool MMQ> struct RawSum {
  static constexpr bool value = QT == KQ_TYPE_Q4_0 || HalfProd<QT>::value ||
                                ((QT == KQ_TYPE_Q4_K || QT == KQ_TYPE_Q5_K) && MMQ) || (QT == KQ_TYPE_Q5_0 && !MMQ);
};
// the six formats every kernel covers; the others go through the general kernels only
inline bool type_is_core(int type) {
  return type == KQ_TYPE_Q4_0 || type == KQ_TYPE_Q8_0 || type == KQ_TYPE_Q2_K || type == KQ_TYPE_Q4_K ||
         type == KQ_TYPE_Q6_K || type == KQ_TYPE_IQ3_S;
}

inline bool type_geometry(int type, int* blk, int* bytes) {
  switch (type) {
    case KQ_TYPE_Q4_0: *blk = 32; *bytes = 18; return true;
    case KQ_TYPE_Q8_0: *blk = 32; *bytes = 34; return true;
    case KQ_TYPE_Q2_K: *blk = 256; *bytes = 84; return true;
    case KQ_TYPE_Q4_K: *blk = 256; *bytes = 144; return true;
    case KQ_TYPE_Q6_K: *blk = 256; *bytes = 210; return true;
    case KQ_TYPE_IQ3_S: *blk = 256; *bytes = 110; return true;
    case KQ_TYPE_Q4_1: *blk = 32; *bytes = 20; return true;
    case KQ_TYPE_Q5_0: *blk = 32; *bytes = 22; return true;
    case KQ_TYPE_Q5_1: *blk = 32; *bytes = 24; return true;
    case KQ_TYPE_Q3_K: *blk = 256; *bytes = 110; return true;
    case KQ_TYPE_Q5_K: *blk = 256; *bytes = 176; return true;
    case KQ_TYPE_IQ4_NL: *blk = 32; *bytes = 18; return true;
    case KQ_TYPE_IQ4_XS: *blk = 256; *bytes = 136; return true;
    default: return false;
  }
}
inline int type_group(int type) { return (type == KQ_TYPE_Q2_K || type == KQ_TYPE_Q6_K || type == KQ_TYPE_Q3_K) ? 16 : 32; }

// ------------------------------------------------------------------ quantized activation scratch
// Activations are quantized to q8_1 (gguf_kernel.cu:32-69 of the reference) into a split layout:
//   ds    half2 [m][kpad/32]        {d, raw fp32 block sum rounded to fp16}
//   qs    int8  [m][kpad]           codes, token-major
// and, for the tensor-core GEMV, per-token scale tables transposed to [token tile][block][16 tokens]
// (tokens beyond m hold zeros) so a K-range of them is one contiguous bulk copy into shared memory:
//   dT    float [mt][kpad/32][16]   d as fp32
//   z32   float [mt][kpad/32][16]   d * (sum of the 32 codes)      (min term, MMVQ flavour)
//   zs8   float [mt][kpad/32][16]   the fp16 raw sum as fp32        (min term of Q4_0 and MMQ-flavoured Q4_K)
//   z16   float [mt][kpad/16][16]   d * (sum of 16 codes)           (min term of Q2_K)
//   qsp   int8  [m][kpad/64][80]    the codes again, 16 bytes of padding after every 64 (bank-conflict-free
//                                   16-byte reads by lanes that are 64 codes apart)
//   xh    half  [m][kpad]           d * code rounded to fp16: the B operand of the tensor-core GEMM
//   s8h   half  [m][kpad/32]        the fp16 raw block sums alone (second B operand of the GEMM)
//   z32r  float [m][kpad/32]        same values as z32, token-major (row-streaming kernel)
//   z16r  float [m][kpad/16]        same values as z16, token-major
//   qsu   bytes [mt][kpad/256][6656]  per unit of 256 weights everything the tensor-memory decode kernel stages for it,
//                                   contiguous (one bulk copy): the codes in the tensor core's K-major core-matrix
//                                   order [16 chunks of 16 weights][16 tokens][16] (4096 B), then float [8 blocks][16
//                                   tokens] of d8 (512 B), of d8 * code sum (512 B), of the raw fp16 sum (512 B), and
//                                   float [16 half blocks][16 tokens] of d8 * code sum per 16 weights (1024 B)
//   part  float [4][16][n]          split-K partial sums of one 16-token pass
//   cnt   int   [KQ_CNT_SLOTS]      split-K arrival counters, one per 8-row tile (the quantizer zeroes the first
//                                   ceil(n/8) of them, the kernel that used them resets them)
//   status int  [64]                device-side error word (bounded waits that gave up)
// Only `part` (which needs no initialisation) and the total depend on n, and `part` comes last: a scratch prepared
// for n_max rows is laid out identically for every weight tensor of n <= n_max rows that shares it.
constexpr int KQ_UNIT_TABLE = 4096 + 3 * 512 + 1024;   // bytes of qsu per (16-token pass, 256 weights)
constexpr int KQ_PART_SLOTS = 4;      // partial-sum slots of a split row tile
constexpr int KQ_CNT_SLOTS = 65536;   // 8-row tiles a split-K launch may have (n <= 524288); larger n runs unsplit
struct Q8Layout {
  int64_t kpad, mt;
  size_t off_ds, off_qs, off_qsp, off_xh, off_s8h, off_dT, off_z32, off_zs8, off_z16, off_z32r, off_z16r, off_qsu, off_part, off_cnt, off_status, off_w16, total;
  int64_t w16_stride;   // halves per row of the Q4_0 coefficient table (0: none)
};
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline Q8Layout q8_layout(int64_t m, int64_t n, int64_t k, int type = 0) {
  Q8Layout L;
  L.kpad = (k + 511) / 512 * 512;
  L.mt = (m + 15) / 16;
  const size_t nb = (size_t)L.kpad / 32;
  size_t p = 0;
  L.off_status = p; p = align_up(p + 256, 256);
  L.off_cnt = p;    p = align_up(p + (size_t)KQ_CNT_SLOTS * 4, 256);
  L.off_ds = p;     p = align_up(p + (size_t)m * nb * 4, 256);
  L.off_qs = p;     p = align_up(p + (size_t)m * L.kpad, 256);
  L.off_qsp = p;    p = align_up(p + (size_t)m * (L.kpad / 64) * 80, 256);
  L.off_xh = p;     p = align_up(p + (size_t)m * L.kpad * 2, 1024);
  L.off_s8h = p;    p = align_up(p + (size_t)m * nb * 2, 1024);
  L.off_dT = p;     p = align_up(p + (size_t)L.mt * nb * 64, 256);
  L.off_z32 = p;    p = align_up(p + (size_t)L.mt * nb * 64, 256);
  L.off_zs8 = p;    p = align_up(p + (size_t)L.mt * nb * 64, 256);
  L.off_z16 = p;    p = align_up(p + (size_t)L.mt * nb * 128, 256);
  L.off_z32r = p;   p = align_up(p + (size_t)m * nb * 4, 256);
  L.off_z16r = p;   p = align_up(p + (size_t)m * nb * 8, 256);
  L.off_qsu = p;    p = align_up(p + (size_t)L.mt * (L.kpad / 256) * KQ_UNIT_TABLE, 256);
  L.off_part = p;   p = align_up(p + (size_t)KQ_PART_SLOTS * 16 * n * 4, 256);
  // Q4_0 calls that may go to the tensor-core GEMM: a dense fp16 table [n][k/32 rounded up to 128] of -8 * d per block,
  // written per call, so that the GEMM's correction steps read 128 contiguous bytes per row instead of 64 scattered scales
  L.w16_stride = (type == KQ_TYPE_Q4_0 && m > 16) ? (int64_t)((nb + 127) / 128 * 128) : 0;
  L.off_w16 = p;    p = align_up(p + (size_t)n * L.w16_stride * 2, 256);
  L.total = p;
  return L;
}

struct Q8Ptrs {  // device pointers into one scratch buffer
  __half2* ds; int8_t* qs; int8_t* qsp; __half* xh; __half* s8h; float *dT, *z32, *zs8, *z16, *z32r, *z16r, *part; int8_t* qsu; int *cnt, *status;
  __half* w16; int64_t w16_stride;   // Q4_0 coefficient table of the GEMM's correction steps (null: none)
  int64_t kpad; int ncnt;
};
inline Q8Ptrs q8_ptrs(void* scratch, const Q8Layout& L, int64_t n) {
  uint8_t* s = (uint8_t*)scratch;
  Q8Ptrs P;
  P.ds = (__half2*)(s + L.off_ds); P.qs = (int8_t*)(s + L.off_qs); P.qsp = (int8_t*)(s + L.off_qsp); P.xh = (__half*)(s + L.off_xh); P.s8h = (__half*)(s + L.off_s8h);
  P.dT = (float*)(s + L.off_dT); P.z32 = (float*)(s + L.off_z32); P.zs8 = (float*)(s + L.off_zs8);
  P.z16 = (float*)(s + L.off_z16); P.z32r = (float*)(s + L.off_z32r); P.z16r = (float*)(s + L.off_z16r);
  P.part = (float*)(s + L.off_part);
  P.w16 = L.w16_stride ? (__half*)(s + L.off_w16) : nullptr; P.w16_stride = L.w16_stride;
  // the unit tables are only written (and read) while the tensor-memory decode kernel is switched on: set the option
  // before the activations are prepared
  P.qsu = (options().umma || options().gemv_impl == 8) ? (int8_t*)(s + L.off_qsu) : nullptr;
  P.cnt = (int*)(s + L.off_cnt); P.status = (int*)(s + L.off_status);
  P.kpad = L.kpad;
  const int64_t tiles = (n + 7) / 8;
  P.ncnt = (int)(tiles < KQ_CNT_SLOTS ? tiles : KQ_CNT_SLOTS);
  return P;
}

// Bulk-copy window of the weight bytes [ga, ge): cp.async.bulk moves 16-byte units between 16-byte aligned addresses,
// so the staged window starts at ga rounded down and ends at ge rounded up.  The streaming kernels are only ever given
// a 16-byte aligned tensor base and a row count whose total size is a multiple of 16 bytes (stream_rows below), so a
// window never reaches outside the tensor: rounding only ever takes in bytes of a neighbouring row.
struct CopyWindow {
  uintptr_t a0;    // start of the bulk copy (16-byte aligned)
  uint32_t lead;   // ga - a0: where the wanted bytes start inside the staged window
  uint32_t bulk;   // bytes of the bulk copy (a multiple of 16)
};
__host__ __device__ inline CopyWindow copy_window(uintptr_t ga, uintptr_t ge) {
  CopyWindow w;
  w.a0 = ga & ~(uintptr_t)15;
  w.lead = (uint32_t)(ga - w.a0);
  w.bulk = (uint32_t)(((ge + 15) & ~(uintptr_t)15) - w.a0);
  return w;
}
// Rows of an n-row tensor the streaming kernels may take: the largest count <= n whose byte size is a multiple of 16
// (row sizes are even, so at most 7 rows are left over); the remaining rows go to the general kernel, which reads
// with plain loads and exact bounds.
inline int64_t stream_rows(int64_t n, int64_t rowbytes) {
  int64_t r = n;
  while (r > 0 && (r * rowbytes) % 16) --r;
  return r;
}

// kernels (defined in the .cu files)
// P may be null (then only the reference 36-byte block layout `wire36` is written)
int launch_quantize(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x,
                    const Q8Ptrs* P, void* wire36, int64_t kpad, cudaStream_t st, int wait_arrival = 0);
int launch_prepare_rmsnorm(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, const void* gamma, float eps,
                           void* y_norm, const Q8Ptrs& P, cudaStream_t st, int wait_arrival = 0);
int launch_prepare_swiglu(const void* gate_up, int x_dtype, int64_t m, int64_t k, int64_t stride_gu, const Q8Ptrs& P,
                          cudaStream_t st, int wait_arrival = 0);
constexpr int KQ_MOE_BLOCK = 8;   // slots per block of expert-sorted tokens (what kq_moe_block_size reports)
int launch_moe(const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* ds, const void* qs, int64_t kpad,
               int64_t tokens, int top_k, const int32_t* ids, int64_t nslots, const int32_t* expert_ids,
               const int32_t* num_post_padded, bool block, void* y, int y_dtype, int64_t stride_y, cudaStream_t st);
int launch_gemv_dp4a(const void* W, int type, int64_t n, int64_t k, const void* ds, const void* qs,
                     int64_t kpad, int64_t m, void* y, int y_dtype, int64_t stride_y, bool mmq,
                     int32_t* dbg_dots, int32_t* dbg_sums, cudaStream_t st);
// tensor-core GEMV; returns KQ_EUNSUPPORTED (without setting an error) when the shape/alignment is not
// covered, so the caller can fall back to the dp4a kernel
bool gemv_mma_supported(const void* W, int type, int64_t n, int64_t k);
bool gemv_rows_only(int type, int64_t n, int64_t k, int64_t m);
int launch_gemv_mma(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m, void* y,
                    int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st, const void* fuse_x = nullptr,
                    int x_dtype = 0, int64_t stride_x = 0);
// Fused all-gather of a row(N)-sharded layer: where the shared-stage kernel writes its outputs (every rank's [M, N]
// buffer, this rank's columns from col0 on) and the flag arrays of the hand-shake that ends the kernel.
struct GatherArgs {
  void* peer_y[8];
  uint32_t* peer_flags[8];
  uint32_t* epoch;
  uint32_t* done;
  int* status;
  int slot, rank, world;
  int64_t col0;
  int ll;               // 1: outputs only, no hand-shake (the consumer polls against the sentinel)
  void* reset;          // ll: local buffer to refill with the sentinel, or null
  size_t reset_bytes;   // a multiple of 16
};
bool gemv_tile_supported(const void* W, int type, int64_t n, int64_t k, int mtok);
int gemv_tile_splits(int type, int64_t n, int64_t k, int mtok);
int launch_gemv_tile(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m0, int mcount, void* y,
                     int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st, const GatherArgs* ga = nullptr);
bool gemv_umma_supported(const void* W, int type, int64_t n, int64_t k);
int launch_gemv_umma(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m0, int mcount, void* y,
                     int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st);
bool gemv_kres_supported(const void* W, int type, int64_t n, int64_t k, int mtok);
int gemv_kres_splits(int type, int64_t n, int64_t k, int mtok);
int launch_gemv_kres(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m0, int mcount, void* y,
                     int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st);
int launch_wait_arrival(const void* buf, size_t bytes, int elem_bytes, int* status, cudaStream_t st);
int arrival_status(int* failed, int clear);
int launch_p2p_allgather(const void* src, size_t bytes, int64_t rows, size_t dst_stride, void* const* peer_dst,
                         uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* done, int slot, int rank, int world,
                         int* status, cudaStream_t st, size_t src_stride = 0);
bool gemm_tc_supported(const void* W, int type, int64_t n, int64_t k);
bool gemm_tc_staged(int type);   // the format's wire bytes reach the unpacking threads through shared memory
int launch_gemm_tc(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m, void* y, int y_dtype,
                   int64_t stride_y, bool mmq, cudaStream_t st);
int launch_dequantize(const void* W, int type, int64_t count, void* out, int out_dtype, cudaStream_t st,
                      const int64_t* ids = nullptr, int64_t k = 0, int64_t nrows = 0, int f32math = 0);

#ifdef __CUDACC__
// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with launch_pdl() may start while its predecessor in the stream is still running.  It must
// call pdl_wait() before it touches anything the predecessor wrote (or writes anything the predecessor may
// still read); what it does before that (barrier set-up, prefetch of the weights, which no kernel of this
// library writes) overlaps the predecessor's tail.  pdl_trigger() lets the successor start as early as possible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------ device helpers
__device__ __forceinline__ uint32_t ld_u16x2(const uint8_t* p) {
  // 32 bits from a 2-byte aligned address (wire blocks of 18/34/110/210 bytes are only 2-aligned)
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
  return (uint32_t)q[0] | ((uint32_t)q[1] << 16);
}
__device__ __forceinline__ uint32_t ld_u32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ float ld_h(const uint8_t* p) {
  return __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(p)));
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// per-byte (v - 32) for bytes in 0..63, no carries between bytes
__device__ __forceinline__ uint32_t sub32_bytes(uint32_t v) {
  return ((v | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
}
// bits 0..3 of `nib` -> 0xFF in byte j if bit j is set
__device__ __forceinline__ uint32_t nibble_to_bytemask(uint32_t nib) {
  uint32_t m = (nib * 0x01010101u) & 0x08040201u;
  uint32_t hb = ((m | 0x80808080u) - 0x01010101u) & 0x80808080u;
  return (hb >> 7) * 0xFFu;
}
// negate the bytes of g (each 4..62) selected by mask (0xFF / 0x00 per byte)
__device__ __forceinline__ uint32_t negate_bytes(uint32_t g, uint32_t mask) {
  return (g ^ mask) + (mask & 0x01010101u);
}
__device__ __forceinline__ uint32_t iq3s_expand(uint32_t code, uint32_t top) {
  // 12-bit code (4 levels x 3 bits) -> 4 grid bytes: level l<7 -> 8l+4, level 7 -> top
  uint32_t r = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t l = (code >> (3 * j)) & 7u;
    uint32_t b = (l == 7u) ? top : (8u * l + 4u);
    r |= b << (8 * j);
  }
  return r;
}
// per-byte (v - 4) for bytes in 0..7, no carries between bytes
__device__ __forceinline__ uint32_t sub4_bytes(uint32_t v) {
  return ((v | 0x80808080u) - 0x04040404u) ^ 0x80808080u;
}
// four 4-bit indices (low nibble of each byte of x) -> the four int8 code values of IQ4_NL / IQ4_XS
// (kvalues_iq4nl, ggml-common.h:1060: -127 -104 -83 -65 -49 -35 -22 -10 1 13 25 38 53 69 89 113), by two byte permutes
// over the table halves and a per-byte select on bit 3
__device__ __forceinline__ uint32_t iq4nl_lookup(uint32_t x) {
  const uint32_t sel = (x & 0x7u) | ((x >> 4) & 0x70u) | ((x >> 8) & 0x700u) | ((x >> 12) & 0x7000u);
  const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel);   // entries 0..7
  const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, sel);   // entries 8..15
  const uint32_t m = ((x >> 3) & 0x01010101u) * 0xFFu;
  return (lo & ~m) | (hi & m);
}
// bits 0..3 of `nib` -> 0x10 in byte j if bit j is set (the fifth bit of four 5-bit codes)
__device__ __forceinline__ uint32_t nibble_to_bit4(uint32_t nib) {
  return ((nib * 0x00204081u) & 0x01010101u) << 4;
}
#ifndef KQ_IQ3S_TOP
#define KQ_IQ3S_TOP 62  // top magnitude byte of the codebook as the reference's CUDA table has it
#endif

// One 32-weight sub-block in the integer-dot domain.
//   v[8]   int8x4 words, word i = weights 4i..4i+3 of the sub-block (same order as the activations)
//   wa[h]  scale of group h (h = 0 for 32-weight groups; h = 0,1 for 16-weight groups = words 0-3 / 4-7)
//   wb[h]  min coefficient of group h (types with HAS_MIN)
// contribution to y:  sum_h  wa[h] * d8 * I_h  -  wb[h] * z_h
//   z_h = d8 * S_h (sum of activation codes) or, for Q4_0 and MMQ-flavoured Q4_K, the fp16 raw sum.
struct SubBlock {
  uint32_t v[8];
  float wa[2];
  float wb[2];
};

// row: first byte of the weight row; sb: 32-weight sub-block index along k; grid: 512-entry IQ3_S table
template <int QT>
__device__ __forceinline__ void decode_subblock(const uint8_t* __restrict__ row, int sb,
                                                const uint32_t* __restrict__ grid, SubBlock& o) {
  if constexpr (QT == KQ_TYPE_Q4_0) {
    const uint8_t* b = row + (size_t)sb * 18;
    const float d = ld_h(b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t w = ld_u16x2(b + 2 + 4 * i);
      o.v[i] = w & 0x0F0F0F0Fu;
      o.v[i + 4] = (w >> 4) & 0x0F0F0F0Fu;
    }
    o.wa[0] = d; o.wb[0] = 8.0f * d; o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_Q8_0) {
    const uint8_t* b = row + (size_t)sb * 34;
    const float d = ld_h(b);
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = ld_u16x2(b + 2 + 4 * i);
    o.wa[0] = d; o.wb[0] = 0.f; o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_Q2_K) {
    const uint8_t* b = row + (size_t)(sb >> 3) * 84;
    const int j = sb & 7, n = j >> 2, jj = j & 3;
    const float d = ld_h(b + 80), dmin = ld_h(b + 82);
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = (ld_u32(b + 16 + 32 * n + 4 * i) >> (2 * jj)) & 0x03030303u;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t s = b[2 * j + h];
      o.wa[h] = d * (float)(s & 15u);
      o.wb[h] = dmin * (float)(s >> 4);
    }
  } else if constexpr (QT == KQ_TYPE_Q4_K) {
    const uint8_t* b = row + (size_t)(sb >> 3) * 144;
    const int j = sb & 7, il = j >> 1, e = j & 1;
    const float d = ld_h(b), dmin = ld_h(b + 2);
    const uint8_t* q = b + 4;
    uint32_t sc, mn;
    if (j < 4) { sc = q[j] & 63u; mn = q[j + 4] & 63u; }
    else { sc = (q[j + 4] & 15u) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = (ld_u32(b + 16 + 32 * il + 4 * i) >> (4 * e)) & 0x0F0F0F0Fu;
    o.wa[0] = d * (float)sc; o.wb[0] = dmin * (float)mn; o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_Q6_K) {
    const uint8_t* b = row + (size_t)(sb >> 3) * 210;
    const int j = sb & 7, ip = j >> 2, q4 = j & 3;
    const float d = ld_h(b + 208);
    const uint8_t* ql = b + 64 * ip + 32 * (q4 & 1);
    const uint8_t* qh = b + 128 + 32 * ip;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t lo = (ld_u16x2(ql + 4 * i) >> (4 * (q4 >> 1))) & 0x0F0F0F0Fu;
      uint32_t hi = (ld_u16x2(qh + 4 * i) >> (2 * q4)) & 0x03030303u;
      o.v[i] = sub32_bytes(lo | (hi << 4));
    }
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192 + 8 * ip + 2 * q4);
    o.wa[0] = d * (float)sc[0]; o.wa[1] = d * (float)sc[1]; o.wb[0] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_IQ3_S) {
    const uint8_t* b = row + (size_t)(sb >> 3) * 110;
    const int ib = sb & 7;
    const float d = ld_h(b);
    // blocks are 2-byte aligned: the sub-block's 8 index bytes and 4 sign bytes as 16-bit loads (6 instead of 12 byte loads)
    const uint16_t* qs16 = reinterpret_cast<const uint16_t*>(b + 2 + 8 * ib);
    const uint32_t qh = b[66 + ib];
    const uint16_t* sg16 = reinterpret_cast<const uint16_t*>(b + 74 + 4 * ib);
    const uint32_t sgw = (uint32_t)sg16[0] | ((uint32_t)sg16[1] << 16);
#pragma unroll
    for (int il = 0; il < 4; ++il) {
      const uint32_t q2 = qs16[il];
      const uint32_t i1 = (q2 & 255u) | ((qh << (8 - 2 * il)) & 256u);
      const uint32_t i2 = (q2 >> 8) | ((qh << (7 - 2 * il)) & 256u);
      const uint32_t s = (sgw >> (8 * il)) & 255u;
      o.v[2 * il] = negate_bytes(grid[i1], nibble_to_bytemask(s & 15u));
      o.v[2 * il + 1] = negate_bytes(grid[i2], nibble_to_bytemask(s >> 4));
    }
    const uint32_t s4 = (b[106 + (ib >> 1)] >> (4 * (ib & 1))) & 15u;
    o.wa[0] = d * (0.5f + (float)s4) * 0.5f; o.wb[0] = 0.f; o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_Q4_1) {            // {half d, half m, qs[16]}: w = d*q + m
    const uint8_t* b = row + (size_t)sb * 20;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = ld_u32(b + 4 + 4 * i);
      o.v[i] = w & 0x0F0F0F0Fu;
      o.v[i + 4] = (w >> 4) & 0x0F0F0F0Fu;
    }
    o.wa[0] = ld_h(b); o.wb[0] = -ld_h(b + 2); o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_Q5_0 || QT == KQ_TYPE_Q5_1) {   // {half d, [half m,] qh[4], qs[16]}: 5-bit codes
    constexpr int HDR = QT == KQ_TYPE_Q5_0 ? 2 : 4;
    const uint8_t* b = row + (size_t)sb * (QT == KQ_TYPE_Q5_0 ? 22 : 24);
    const uint32_t qh = ld_u16x2(b + HDR);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = ld_u16x2(b + HDR + 4 + 4 * i);
      o.v[i] = (w & 0x0F0F0F0Fu) | nibble_to_bit4((qh >> (4 * i)) & 15u);
      o.v[i + 4] = ((w >> 4) & 0x0F0F0F0Fu) | nibble_to_bit4((qh >> (16 + 4 * i)) & 15u);
    }
    const float d = ld_h(b);
    if constexpr (QT == KQ_TYPE_Q5_0) { o.wa[0] = d; o.wb[0] = 16.0f * d; }
    else { o.wa[0] = d; o.wb[0] = -ld_h(b + 2); }
    o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_Q3_K) {             // {hmask[32], qs[64], scales[12], half d}: 3-bit codes - 4
    const uint8_t* b = row + (size_t)(sb >> 3) * 110;
    const int j = sb & 7, n = j >> 2, jj = j & 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t lo = (ld_u16x2(b + 32 + 32 * n + 4 * i) >> (2 * jj)) & 0x03030303u;
      const uint32_t hb = (ld_u16x2(b + 4 * i) >> (4 * n + jj)) & 0x01010101u;
      o.v[i] = sub4_bytes(lo | (hb << 2));
    }
    const float d = ld_h(b + 108);
    const uint8_t* sc = b + 96;
#pragma unroll
    for (int h = 0; h < 2; ++h) {                        // 6-bit scales of the two 16-weight groups (dequantize.cuh:139-142)
      const int is = 2 * j + h;
      int us;
      if (is < 4) us = (sc[is] & 15) | (((sc[is + 8] >> 0) & 3) << 4);
      else if (is < 8) us = (sc[is] & 15) | (((sc[is + 4] >> 2) & 3) << 4);
      else if (is < 12) us = (sc[is - 8] >> 4) | (((sc[is] >> 4) & 3) << 4);
      else us = (sc[is - 8] >> 4) | (((sc[is - 4] >> 6) & 3) << 4);
      o.wa[h] = d * (float)(us - 32);
      o.wb[h] = 0.f;
    }
  } else if constexpr (QT == KQ_TYPE_Q5_K) {             // {half d, half dmin, scales[12], qh[32], qs[128]}
    const uint8_t* b = row + (size_t)(sb >> 3) * 176;
    const int j = sb & 7, il = j >> 1, e = j & 1;
    const float d = ld_h(b), dmin = ld_h(b + 2);
    const uint8_t* q = b + 4;
    uint32_t sc, mn;
    if (j < 4) { sc = q[j] & 63u; mn = q[j + 4] & 63u; }
    else { sc = (q[j + 4] & 15u) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t lo = (ld_u32(b + 48 + 32 * il + 4 * i) >> (4 * e)) & 0x0F0F0F0Fu;
      const uint32_t hb = (ld_u32(b + 16 + 4 * i) >> j) & 0x01010101u;
      o.v[i] = lo | (hb << 4);
    }
    o.wa[0] = d * (float)sc; o.wb[0] = dmin * (float)mn; o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_IQ4_NL) {           // {half d, qs[16]}: 4-bit indices into 16 code values
    const uint8_t* b = row + (size_t)sb * 18;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = ld_u16x2(b + 2 + 4 * i);
      o.v[i] = iq4nl_lookup(w & 0x0F0F0F0Fu);
      o.v[i + 4] = iq4nl_lookup((w >> 4) & 0x0F0F0F0Fu);
    }
    o.wa[0] = ld_h(b); o.wb[0] = 0.f; o.wa[1] = 0.f; o.wb[1] = 0.f;
  } else if constexpr (QT == KQ_TYPE_IQ4_XS) {           // {half d, u16 scales_h, scales_l[4], qs[128]}
    const uint8_t* b = row + (size_t)(sb >> 3) * 136;
    const int ib = sb & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w = ld_u32(b + 8 + 16 * ib + 4 * i);
      o.v[i] = iq4nl_lookup(w & 0x0F0F0F0Fu);
      o.v[i + 4] = iq4nl_lookup((w >> 4) & 0x0F0F0F0Fu);
    }
    const uint32_t sh = *reinterpret_cast<const uint16_t*>(b + 2);
    const int ls = (int)(((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15u) | (((sh >> (2 * ib)) & 3u) << 4));
    o.wa[0] = ld_h(b) * (float)(ls - 32); o.wb[0] = 0.f; o.wa[1] = 0.f; o.wb[1] = 0.f;
  }
}
#endif  // __CUDACC__

}  // namespace kq
