// C ABI of libkq (see include/kq_gguf.h): argument validation, scratch carving, kernel selection.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "kq_common.cuh"

namespace kq {

static thread_local char t_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return KQ_ECUDA;
}

Options& options() {
  static Options o = {0, 3, 81, 2, 1, 0, 0, 1, 1, 0, 1, 1, 0, 1, 24, 1, 1, 1};
  return o;
}

int sm_count() {
  static int counts[64] = {0};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev >= 0 && counts[dev] > 0) return counts[dev];
  if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0) counts[dev] = n;
  return n;
}

static bool dtype_ok(int dt) { return dt == KQ_F32 || dt == KQ_F16 || dt == KQ_BF16; }
static size_t dtype_size(int dt) { return dt == KQ_F32 ? 4 : 2; }

struct Problem {
  int blk, bytes;
  int64_t rowbytes;
  Q8Layout L;
};

// need_w / need_x: the prepare / prepared entry points pass only one of the two operands
static int validate(const char* fn, const void* W, int type, int64_t n, int64_t k, const void* x, int x_dtype,
                    int64_t m, int64_t stride_x, const void* scratch, size_t scratch_bytes, Problem& p,
                    bool need_w = true, bool need_x = true) {
  if (!type_geometry(type, &p.blk, &p.bytes)) {
    set_error("%s: GGML type %d is not supported (supported: 2 Q4_0, 3 Q4_1, 6 Q5_0, 7 Q5_1, 8 Q8_0, 10 Q2_K, 11 Q3_K, 12 Q4_K, "
              "13 Q5_K, 14 Q6_K, 20 IQ4_NL, 21 IQ3_S, 23 IQ4_XS)", fn, type);
    return KQ_EUNSUPPORTED;
  }
  if (need_x && !dtype_ok(x_dtype)) { set_error("%s: unsupported activation dtype %d", fn, x_dtype); return KQ_EUNSUPPORTED; }
  if (n <= 0 || k <= 0 || m <= 0) { set_error("%s: n, k, m must be positive (n=%lld k=%lld m=%lld)", fn, (long long)n, (long long)k, (long long)m); return KQ_EINVAL; }
  if (k % p.blk) { set_error("%s: k=%lld is not a multiple of the block size %d", fn, (long long)k, p.blk); return KQ_EINVAL; }
  if (n > 0x7fffffff / 2 || k > (1 << 24) || m > (1 << 20)) { set_error("%s: size out of range", fn); return KQ_ELIMIT; }
  if ((need_w && !W) || (need_x && !x)) { set_error("%s: null pointer", fn); return KQ_EINVAL; }
  if (need_x && stride_x < k) { set_error("%s: stride_x=%lld < k=%lld", fn, (long long)stride_x, (long long)k); return KQ_EINVAL; }
  const uintptr_t wa = (uintptr_t)W;
  const int need = (p.bytes % 4 == 0) ? 4 : 2;
  if (wa % need) { set_error("%s: weight pointer must be %d-byte aligned for this type", fn, need); return KQ_EINVAL; }
  if (need_x && (uintptr_t)x % dtype_size(x_dtype)) { set_error("%s: misaligned activation pointer", fn); return KQ_EINVAL; }
  p.rowbytes = k / p.blk * p.bytes;
  p.L = q8_layout(m, n, k, type);
  if (!scratch || (uintptr_t)scratch % 256) { set_error("%s: scratch must be non-null and 256-byte aligned", fn); return KQ_ESCRATCH; }
  if (scratch_bytes < p.L.total) { set_error("%s: scratch too small (%zu < %zu)", fn, scratch_bytes, p.L.total); return KQ_ESCRATCH; }
  return KQ_OK;
}

// tcgen05 GEMM or passes of the integer GEMV?  From gemm_min_m tokens on always the GEMM.  Below that (17+ tokens,
// i.e. two or more GEMV passes) the GEMM takes the call when its time, flat in m up to 256 tokens, beats the passes.
// Measured (us, whole call, GEMV passes at 17 / 33 / 48 / 80 tokens against the GEMM):
//   Q4_K 17408x5120 (136 row tiles)  42 / 64 / 71 / 116   against  38
//   Q8_0  8192x5120  (64)            34 / 53 / 61 /  99   against  54      Q2_K 8192x2048 (64)  21 / 31 / 35 / 57  against 23
//   Q4_0  8192x5120  (64)            36 / 60 / 75 / 122   against  58      Q4_0 17408x5120 (136)  50 / 75 / .. / ..  against 68
//   Q8_0  5120x5120  (40)            26 / 42 / 50 /  79   against  54      Q4_K 4096x4096 (32)  17 / 25 / 30 / 48  against 30
//   Q6_K  5120x17408 (40, long K)    57 / 93 / 111 / 184  against 175
static bool gemm_wanted(int type, int64_t n, int64_t k, int64_t m) {
  const Options& o = options();
  if (o.gemv_impl != 0) return false;
  if (m >= o.gemm_min_m) return true;
  if (!o.gemm_small_m || m <= 16 || !gemm_tc_staged(type) || (k % 256) != 0) return false;
  const int64_t tiles = (n + 127) / 128;
  const bool q40 = type == KQ_TYPE_Q4_0, q6k = type == KQ_TYPE_Q6_K;   // more time per K step than the others
  if (tiles >= 120) return m >= (q40 ? 33 : 17);
  if (tiles >= 60) return m >= (q6k ? 49 : 33);
  if (tiles >= 30) return !q6k && m >= 49;
  return false;
}

// A preparation does not know which weight tensors (type, n) will be multiplied against it: it writes the GEMM's fp16
// operands whenever some tensor could take the GEMM at this token count.
static bool prepare_writes_gemm_operands(int64_t m) {
  const Options& o = options();
  return o.gemv_impl == 0 && (m >= o.gemm_min_m || (o.gemm_small_m && m > 16));
}

static int mul_mat(const char* fn, bool mmq, const void* W, int type, int64_t n, int64_t k, const void* x,
                   int x_dtype, int64_t m, int64_t stride_x, void* y, int y_dtype, int64_t stride_y, void* scratch,
                   size_t scratch_bytes, void* stream, bool need_w = true, bool need_x = true, int wait_arrival = 0) {
  t_err[0] = 0;
  Problem p;
  int rc = validate(fn, W, type, n, k, x, x_dtype, m, stride_x, scratch, scratch_bytes, p, need_w, need_x);
  if (rc) return rc;
  if (!need_w) {
    Q8Ptrs P = q8_ptrs(scratch, p.L, n);
    if (!prepare_writes_gemm_operands(m)) P.xh = nullptr;
    return launch_quantize(x, x_dtype, m, k, stride_x, &P, nullptr, p.L.kpad, (cudaStream_t)stream, wait_arrival);
  }
  if (mmq && (type == KQ_TYPE_IQ3_S || type == KQ_TYPE_IQ4_NL || type == KQ_TYPE_IQ4_XS)) {
    set_error("%s: the i-matrix formats have no MMQ kernel (use dequantize + matmul or mul_mat_vec)", fn);
    return KQ_EUNSUPPORTED;
  }
  if (!dtype_ok(y_dtype)) { set_error("%s: unsupported output dtype %d", fn, y_dtype); return KQ_EUNSUPPORTED; }
  if (!y || stride_y < n) { set_error("%s: bad output (null or stride_y < n)", fn); return KQ_EINVAL; }
  if ((uintptr_t)y % dtype_size(y_dtype)) { set_error("%s: misaligned output pointer", fn); return KQ_EINVAL; }
  cudaStream_t st = (cudaStream_t)stream;
  Q8Ptrs P = q8_ptrs(scratch, p.L, n);
  const int impl = options().gemv_impl;
  const bool gemm = gemm_wanted(type, n, k, m) && gemm_tc_supported(W, type, n, k);
  if (!gemm && need_x) P.xh = nullptr;   // the fp16 copy of the activations is only written for the GEMM
  // 1-2 tokens on the row-streaming kernel: its consumer warps quantize x themselves while the first weights arrive
  // (measured: it pays when all (token, 32-block) pairs fit one pass of the 512 consumer lanes and the matrix is big
  // enough for the ~2 us of quantization to hide behind the pipeline fill: 16.9 -> 15.4 us on Q4_K 17408x5120 at one
  // token; a second pass, or a matrix of a few MB, makes it slower than the separate launch)
  const bool fuse_fits = options().fuse_q8 == 2 || (m * (k / 32) <= 512 && n * p.rowbytes >= (32ll << 20));   // 2: wherever it can run (tests)
  const bool fuse = x && !gemm && options().fuse_q8 && m <= 2 && fuse_fits && stream_rows(n, p.rowbytes) == n &&
                    impl != 1 && gemv_rows_only(type, n, k, m) && gemv_mma_supported(W, type, n, k);
  if (fuse) return launch_gemv_mma(W, type, n, k, P, m, y, y_dtype, stride_y, mmq, st, x, x_dtype, stride_x);
  if (x) {
    Q8Ptrs Pq = P;
    if (gemm) {   // the GEMM reads only the fp16 activations and raw block sums: skip the GEMV-side tables
      Pq.qs = nullptr; Pq.qsp = nullptr; Pq.ds = nullptr; Pq.dT = nullptr; Pq.qsu = nullptr;
    }
    rc = launch_quantize(x, x_dtype, m, k, stride_x, &Pq, nullptr, p.L.kpad, st);
    if (rc) return rc;
  }
  if (gemm) return launch_gemm_tc(W, type, n, k, P, m, y, y_dtype, stride_y, mmq, st);
  if (impl != 1 && gemv_mma_supported(W, type, n, k)) {
    // the streaming kernels take the rows whose total size is a multiple of 16 bytes (all of them for every even n);
    // up to 7 rows at the end of an odd-sized tensor go to the general kernel, so nothing is read past the tensor
    const int64_t ns = stream_rows(n, p.rowbytes);
    if (ns > 0) {
      rc = launch_gemv_mma(W, type, ns, k, P, m, y, y_dtype, stride_y, mmq, st);
      if (rc) return rc;
    }
    if (ns == n) return KQ_OK;
    return launch_gemv_dp4a((const uint8_t*)W + ns * p.rowbytes, type, n - ns, k, P.ds, P.qs, p.L.kpad, m,
                            (uint8_t*)y + ns * dtype_size(y_dtype), y_dtype, stride_y, mmq, nullptr, nullptr, st);
  }
  if (impl >= 2) { set_error("%s: the streaming GEMV does not cover this shape/alignment", fn); return KQ_EUNSUPPORTED; }
  return launch_gemv_dp4a(W, type, n, k, P.ds, P.qs, p.L.kpad, m, y, y_dtype, stride_y, mmq, nullptr, nullptr, st);
}

}  // namespace kq

using namespace kq;

extern "C" {

const char* kq_last_error(void) { return t_err; }
int kq_abi_version(void) { return 1; }

int kq_block_geometry(int type, int* weights_per_block, int* bytes_per_block) {
  int b, s;
  if (!type_geometry(type, &b, &s)) { set_error("kq_block_geometry: GGML type %d is not supported", type); return KQ_EUNSUPPORTED; }
  if (weights_per_block) *weights_per_block = b;
  if (bytes_per_block) *bytes_per_block = s;
  return KQ_OK;
}

size_t kq_workspace_bytes(int type, int64_t m, int64_t n, int64_t k) {
  int b, s;
  if (!type_geometry(type, &b, &s) || m <= 0 || n <= 0 || k <= 0) return 0;
  return q8_layout(m, n, k, type).total;
}

int kq_quantize_q8_1(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, void* out_blocks, void* stream) {
  t_err[0] = 0;
  if (!x || !out_blocks) { set_error("kq_quantize_q8_1: null pointer"); return KQ_EINVAL; }
  if (m <= 0 || k <= 0 || stride_x < k) { set_error("kq_quantize_q8_1: bad sizes"); return KQ_EINVAL; }
  if (!dtype_ok(x_dtype)) { set_error("kq_quantize_q8_1: unsupported dtype %d", x_dtype); return KQ_EUNSUPPORTED; }
  if ((uintptr_t)out_blocks % 4) { set_error("kq_quantize_q8_1: output must be 4-byte aligned"); return KQ_EINVAL; }
  const int64_t kpad = (k + 511) / 512 * 512;
  return launch_quantize(x, x_dtype, m, k, stride_x, nullptr, out_blocks, kpad, (cudaStream_t)stream);
}

int kq_mul_mat_vec_a8(const void* W, int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m,
                      int64_t stride_x, void* y, int y_dtype, int64_t stride_y, void* scratch, size_t scratch_bytes,
                      void* stream) {
  return mul_mat("kq_mul_mat_vec_a8", false, W, type, n, k, x, x_dtype, m, stride_x, y, y_dtype, stride_y, scratch,
                 scratch_bytes, stream);
}

int kq_mul_mat_a8(const void* W, int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m,
                  int64_t stride_x, void* y, int y_dtype, int64_t stride_y, void* scratch, size_t scratch_bytes,
                  void* stream) {
  return mul_mat("kq_mul_mat_a8", true, W, type, n, k, x, x_dtype, m, stride_x, y, y_dtype, stride_y, scratch,
                 scratch_bytes, stream);
}

int kq_prepare_q8(int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m, int64_t stride_x,
                  void* scratch, size_t scratch_bytes, int flags, void* stream) {
  if (flags & ~KQ_PREP_WAIT_ARRIVAL) { set_error("kq_prepare_q8: unknown flag bits %d", flags); return KQ_EINVAL; }
  if ((flags & KQ_PREP_WAIT_ARRIVAL) && m > 80) { set_error("kq_prepare_q8: arrival polling serves the decode path (m <= 80)"); return KQ_ELIMIT; }
  return mul_mat("kq_prepare_q8", false, nullptr, type, n, k, x, x_dtype, m, stride_x, nullptr, KQ_F32, n, scratch,
                 scratch_bytes, stream, false, true, flags & KQ_PREP_WAIT_ARRIVAL);
}

// shared validation of the fused producers: same checks as kq_prepare_q8, then the scratch pointers
static int prepare_common(const char* fn, int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m, int64_t stride_x,
                          int64_t min_stride, void* scratch, size_t scratch_bytes, Q8Ptrs* P) {
  t_err[0] = 0;
  Problem p;
  int rc = validate(fn, nullptr, type, n, k, x, x_dtype, m, stride_x < k ? k : stride_x, scratch, scratch_bytes, p, false, true);
  if (rc) return rc;
  if (stride_x < min_stride) { set_error("%s: row stride %lld < %lld", fn, (long long)stride_x, (long long)min_stride); return KQ_EINVAL; }
  if (m > 80) { set_error("%s: the fused producers serve the decode path (m <= 80)", fn); return KQ_ELIMIT; }
  *P = q8_ptrs(scratch, p.L, n);
  if (!prepare_writes_gemm_operands(m)) P->xh = nullptr;   // the GEMM's fp16 operands only where some projection may be a GEMM
  return KQ_OK;
}

int kq_prepare_q8_rmsnorm(int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m, int64_t stride_x,
                          const void* gamma, float eps, void* y_norm, void* scratch, size_t scratch_bytes, int flags,
                          void* stream) {
  Q8Ptrs P;
  int rc = prepare_common("kq_prepare_q8_rmsnorm", type, n, k, x, x_dtype, m, stride_x, k, scratch, scratch_bytes, &P);
  if (rc) return rc;
  if (!gamma) { set_error("kq_prepare_q8_rmsnorm: null gamma"); return KQ_EINVAL; }
  if (flags & ~KQ_PREP_WAIT_ARRIVAL) { set_error("kq_prepare_q8_rmsnorm: unknown flag bits %d", flags); return KQ_EINVAL; }
  return launch_prepare_rmsnorm(x, x_dtype, m, k, stride_x, gamma, eps, y_norm, P, (cudaStream_t)stream, flags & KQ_PREP_WAIT_ARRIVAL);
}

int kq_prepare_q8_swiglu(int type, int64_t n, int64_t k, const void* gate_up, int x_dtype, int64_t m, int64_t stride_gu,
                         void* scratch, size_t scratch_bytes, int flags, void* stream) {
  Q8Ptrs P;
  int rc = prepare_common("kq_prepare_q8_swiglu", type, n, k, gate_up, x_dtype, m, stride_gu, 2 * k, scratch, scratch_bytes, &P);
  if (rc) return rc;
  if (flags & ~KQ_PREP_WAIT_ARRIVAL) { set_error("kq_prepare_q8_swiglu: unknown flag bits %d", flags); return KQ_EINVAL; }
  return launch_prepare_swiglu(gate_up, x_dtype, m, k, stride_gu, P, (cudaStream_t)stream, flags & KQ_PREP_WAIT_ARRIVAL);
}

int kq_mul_mat_prepared(const void* W, int type, int64_t n, int64_t k, int64_t m, void* y, int y_dtype,
                        int64_t stride_y, int mmq, void* scratch, size_t scratch_bytes, void* stream) {
  return mul_mat("kq_mul_mat_prepared", mmq != 0, W, type, n, k, nullptr, KQ_F32, m, k, y, y_dtype, stride_y, scratch,
                 scratch_bytes, stream, true, false);
}

// ---------------------------------------------------------------------------------------------- no-allocation variant
// Scratch for kq_mul_mat_vec_a8_static: a file-scope device array, one copy per GPU that loads the library.
// Sized for the stated limits m <= 16, n <= 32768, k <= 32768 (layout of q8_layout at those maxima, rounded up).
constexpr int64_t KQ_STATIC_MAX_M = 16, KQ_STATIC_MAX_N = 32768, KQ_STATIC_MAX_K = 32768;
constexpr size_t KQ_STATIC_BYTES = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[KQ_STATIC_BYTES];

// The array's name is only a host-side handle; kernels need its device address, looked up once per device.
static void* static_scratch_ptr(int* rc) {
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaGetDevice"); return nullptr; }
  if (dev < 0 || dev >= 64) { set_error("kq_mul_mat_vec_a8_static: device index %d out of range", dev); *rc = KQ_ELIMIT; return nullptr; }
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaGetSymbolAddress(g_static_scratch)"); return nullptr; }
    ptrs[dev] = p;
  }
  *rc = KQ_OK;
  return ptrs[dev];
}

int kq_mul_mat_vec_a8_static(const void* W, int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m,
                             int64_t stride_x, void* y, int y_dtype, int64_t stride_y, void* stream) {
  t_err[0] = 0;
  if (m > KQ_STATIC_MAX_M || n > KQ_STATIC_MAX_N || k > KQ_STATIC_MAX_K) {
    set_error("kq_mul_mat_vec_a8_static: size beyond the built-in scratch (limits: m <= %lld, n <= %lld, k <= %lld; got m=%lld n=%lld k=%lld)",
              (long long)KQ_STATIC_MAX_M, (long long)KQ_STATIC_MAX_N, (long long)KQ_STATIC_MAX_K, (long long)m, (long long)n, (long long)k);
    return KQ_ELIMIT;
  }
  if (m > 0 && n > 0 && k > 0 && q8_layout(m, n, k).total > KQ_STATIC_BYTES) {
    set_error("kq_mul_mat_vec_a8_static: internal scratch layout exceeds the built-in array");
    return KQ_ELIMIT;
  }
  int rc = KQ_OK;
  void* scratch = static_scratch_ptr(&rc);
  if (!scratch) return rc;
  return mul_mat("kq_mul_mat_vec_a8_static", false, W, type, n, k, x, x_dtype, m, stride_x, y, y_dtype, stride_y, scratch,
                 KQ_STATIC_BYTES, stream);
}

int kq_read_status_static(int* status) {
  t_err[0] = 0;
  if (!status) { set_error("kq_read_status_static: null pointer"); return KQ_EINVAL; }
  int rc = KQ_OK;
  const uint8_t* scratch = (const uint8_t*)static_scratch_ptr(&rc);
  if (!scratch) return rc;
  // the status word sits at a fixed offset of the layout, whatever sizes the array was last used with
  KQ_CUDA_TRY(cudaMemcpy(status, scratch + q8_layout(1, 1, 32).off_status, sizeof(int), cudaMemcpyDeviceToHost));
  return KQ_OK;
}

int kq_dequantize(const void* W, int type, int64_t count, void* out, int out_dtype, void* stream) {
  t_err[0] = 0;
  int b, s;
  if (!type_geometry(type, &b, &s)) { set_error("kq_dequantize: GGML type %d is not supported", type); return KQ_EUNSUPPORTED; }
  if (!dtype_ok(out_dtype)) { set_error("kq_dequantize: unsupported output dtype %d", out_dtype); return KQ_EUNSUPPORTED; }
  if (count < 0 || count % b) { set_error("kq_dequantize: count=%lld is not a multiple of the block size %d", (long long)count, b); return KQ_EINVAL; }
  if (count == 0) return KQ_OK;
  if (!W || !out) { set_error("kq_dequantize: null pointer"); return KQ_EINVAL; }
  if ((uintptr_t)W % 2 || (uintptr_t)out % 16) { set_error("kq_dequantize: W must be 2-byte and out 16-byte aligned"); return KQ_EINVAL; }
  return launch_dequantize(W, type, count, out, out_dtype, (cudaStream_t)stream);
}

int kq_dequantize_rows(const void* W, int type, int64_t n, int64_t k, const int64_t* row_ids, int64_t count, void* out,
                       int out_dtype, int f32_math, void* stream) {
  t_err[0] = 0;
  int b, s;
  if (!type_geometry(type, &b, &s)) { set_error("kq_dequantize_rows: GGML type %d is not supported", type); return KQ_EUNSUPPORTED; }
  if (!dtype_ok(out_dtype)) { set_error("kq_dequantize_rows: unsupported output dtype %d", out_dtype); return KQ_EUNSUPPORTED; }
  if (n <= 0 || k <= 0 || k % b || count < 0) { set_error("kq_dequantize_rows: k=%lld must be a positive multiple of the block size %d", (long long)k, b); return KQ_EINVAL; }
  if (count == 0) return KQ_OK;
  if (!W || !out || !row_ids) { set_error("kq_dequantize_rows: null pointer"); return KQ_EINVAL; }
  if ((uintptr_t)W % 2 || (uintptr_t)out % 16 || (uintptr_t)row_ids % 8) { set_error("kq_dequantize_rows: W must be 2-byte, out 16-byte, row_ids 8-byte aligned"); return KQ_EINVAL; }
  return launch_dequantize(W, type, count * k, out, out_dtype, (cudaStream_t)stream, row_ids, k, n, f32_math != 0);
}

int kq_debug_group_dots(const void* W, int type, int64_t n, int64_t k, const void* x, int x_dtype, int64_t m,
                        int64_t stride_x, int32_t* dots, int32_t* sums, void* scratch, size_t scratch_bytes,
                        void* stream) {
  t_err[0] = 0;
  Problem p;
  int rc = validate("kq_debug_group_dots", W, type, n, k, x, x_dtype, m, stride_x, scratch, scratch_bytes, p);
  if (rc) return rc;
  if (!dots) { set_error("kq_debug_group_dots: null dots"); return KQ_EINVAL; }
  cudaStream_t st = (cudaStream_t)stream;
  Q8Ptrs P = q8_ptrs(scratch, p.L, n);
  P.xh = nullptr;
  rc = launch_quantize(x, x_dtype, m, k, stride_x, &P, nullptr, p.L.kpad, st);
  if (rc) return rc;
  return launch_gemv_dp4a(W, type, n, k, P.ds, P.qs, p.L.kpad, m, nullptr, KQ_F32, n, false, dots, sums, st);
}

int kq_read_status(int type, int64_t m, int64_t n, int64_t k, const void* scratch, size_t scratch_bytes, int* status) {
  t_err[0] = 0;
  int b, sz;
  if (!type_geometry(type, &b, &sz) || m <= 0 || n <= 0 || k <= 0 || !scratch || !status) { set_error("kq_read_status: bad argument"); return KQ_EINVAL; }
  const Q8Layout L = q8_layout(m, n, k);
  if (scratch_bytes < L.total) { set_error("kq_read_status: scratch too small"); return KQ_ESCRATCH; }
  KQ_CUDA_TRY(cudaMemcpy(status, (const uint8_t*)scratch + L.off_status, sizeof(int), cudaMemcpyDeviceToHost));
  return KQ_OK;
}

int kq_p2p_allgather(const void* src, size_t bytes, void* const* peer_dst, uint32_t* const* peer_flags,
                     uint32_t* epoch, uint32_t* done, int slot, int rank, int world, int* status, void* stream) {
  if (!src || !peer_dst || !peer_flags || !epoch || !done || !status) {
    set_error("kq_p2p_allgather: null pointer argument");
    return KQ_EINVAL;
  }
  return launch_p2p_allgather(src, bytes, 0, 0, peer_dst, peer_flags, epoch, done, slot, rank, world, status, (cudaStream_t)stream);
}

int kq_p2p_allgather_2d(const void* src, int64_t rows, size_t row_bytes, void* const* peer_dst, size_t dst_row_stride,
                        uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* done, int slot, int rank, int world,
                        int* status, void* stream) {
  if (!src || !peer_dst || !peer_flags || !epoch || !done || !status || rows <= 0) {
    set_error("kq_p2p_allgather_2d: null pointer or non-positive row count");
    return KQ_EINVAL;
  }
  return launch_p2p_allgather(src, (size_t)rows * row_bytes, rows, dst_row_stride, peer_dst, peer_flags, epoch, done, slot, rank,
                              world, status, (cudaStream_t)stream);
}

int kq_mul_mat_prepared_gather(const void* W, int type, int64_t n_local, int64_t k, int64_t m, int y_dtype, int mmq,
                               void* scratch, size_t scratch_bytes, void* const* peer_y, int64_t stride_y,
                               uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* done, int slot, int rank,
                               int world, int* peer_status, int wait_in_consumer, void* reset_buf, size_t reset_bytes,
                               int* fused, void* stream) {
  t_err[0] = 0;
  const char* fn = "kq_mul_mat_prepared_gather";
  if (reset_buf && ((uintptr_t)reset_buf % 16 || reset_bytes % 16)) { set_error("%s: reset_buf must be 16-byte aligned and sized", fn); return KQ_EINVAL; }
  if (!wait_in_consumer) { reset_buf = nullptr; reset_bytes = 0; }
  if (fused) *fused = 0;
  if (!peer_y || !peer_flags || !epoch || !done || !peer_status) { set_error("%s: null pointer argument", fn); return KQ_EINVAL; }
  if (world < 1 || world > 8 || rank < 0 || rank >= world || slot < 0) {
    set_error("%s: world %d (max 8), rank %d, slot %d", fn, world, rank, slot);
    return KQ_EINVAL;
  }
  if (!dtype_ok(y_dtype)) { set_error("%s: unsupported output dtype %d", fn, y_dtype); return KQ_EUNSUPPORTED; }
  if (n_local <= 0 || stride_y < (int64_t)world * n_local) { set_error("%s: stride_y < world * n_local", fn); return KQ_EINVAL; }
  const size_t esz = dtype_size(y_dtype);
  uintptr_t bits = (uintptr_t)((size_t)n_local * esz) | (uintptr_t)((size_t)stride_y * esz);
  for (int r = 0; r < world; ++r) {
    if (!peer_y[r] || !peer_flags[r]) { set_error("%s: null buffer or flag pointer for rank %d", fn, r); return KQ_EINVAL; }
    if ((uintptr_t)peer_flags[r] % 4 || (uintptr_t)peer_y[r] % esz) { set_error("%s: misaligned buffer or flag array of rank %d", fn, r); return KQ_EINVAL; }
    bits |= (uintptr_t)peer_y[r];
  }
  Problem p;
  int rc = validate(fn, W, type, n_local, k, nullptr, KQ_F32, m, k, scratch, scratch_bytes, p, true, false);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  Q8Ptrs P = q8_ptrs(scratch, p.L, n_local);
  const int64_t col0 = (int64_t)rank * n_local;
  // one kernel: the shared-stage kernel takes the whole call (<= 16 tokens, all rows streamable) and every 16-byte
  // output store is aligned in every rank's buffer
  const bool one = world > 1 && options().gemv_impl == 0 && !options().no_fused_gather && m <= 16 && (bits & 15) == 0 &&
                   !(mmq && (type == KQ_TYPE_IQ3_S || type == KQ_TYPE_IQ4_NL || type == KQ_TYPE_IQ4_XS)) &&
                   gemv_mma_supported(W, type, n_local, k) && stream_rows(n_local, p.rowbytes) == n_local &&
                   gemv_tile_supported(W, type, n_local, k, (int)m);
  if (one) {
    GatherArgs ga;
    for (int r = 0; r < 8; ++r) { ga.peer_y[r] = r < world ? peer_y[r] : nullptr; ga.peer_flags[r] = r < world ? peer_flags[r] : nullptr; }
    ga.epoch = epoch; ga.done = done; ga.status = peer_status; ga.slot = slot; ga.rank = rank; ga.world = world; ga.col0 = col0;
    ga.ll = wait_in_consumer != 0; ga.reset = reset_buf; ga.reset_bytes = reset_bytes;
    rc = launch_gemv_tile(W, type, n_local, k, P, 0, (int)m, peer_y[rank], y_dtype, stride_y, mmq != 0, st, &ga);
    if (rc == KQ_OK && fused) *fused = 1;
    return rc;
  }
  // two kernels: the usual dispatch writes this rank's columns of its own buffer, the gather kernel pushes them out
  // (with its hand-shake: the consumer's sentinel test then passes at once; the consumed buffer is refilled here)
  if (reset_buf && reset_bytes) KQ_CUDA_TRY(cudaMemsetAsync(reset_buf, 0xFF, reset_bytes, st));
  uint8_t* mine = (uint8_t*)peer_y[rank] + (size_t)col0 * esz;
  rc = mul_mat(fn, mmq != 0, W, type, n_local, k, nullptr, KQ_F32, m, k, mine, y_dtype, stride_y, scratch, scratch_bytes, stream,
               true, false);
  if (rc || world == 1) return rc;
  return launch_p2p_allgather(mine, (size_t)m * n_local * esz, m, (size_t)stride_y * esz, peer_y, peer_flags, epoch, done, slot,
                              rank, world, peer_status, st, (size_t)stride_y * esz);
}

// ---------------------------------------------------------------------------------------------- mixture of experts
static int moe_common(const char* fn, bool block, const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* x,
                      int x_dtype, int64_t tokens, int64_t stride_x, const int32_t* ids, int64_t nslots, const int32_t* expert_ids,
                      const int32_t* num_post_padded, int top_k, void* y, int y_dtype, int64_t stride_y, void* scratch,
                      size_t scratch_bytes, void* stream) {
  t_err[0] = 0;
  if (experts <= 0 || top_k <= 0 || nslots < 0) { set_error("%s: experts, top_k must be positive", fn); return KQ_EINVAL; }
  if (!ids || (block && (!expert_ids || !num_post_padded))) { set_error("%s: null index tensor", fn); return KQ_EINVAL; }
  if (tokens == 0) return KQ_OK;
  Problem p;
  int rc = validate(fn, W, type, n, k, x, x_dtype, tokens, stride_x, scratch, scratch_bytes, p, true, true);
  if (rc) return rc;
  if (block && (type == KQ_TYPE_IQ3_S || type == KQ_TYPE_IQ4_NL || type == KQ_TYPE_IQ4_XS)) {
    set_error("%s: the i-matrix formats have no MMQ kernel (use kq_moe_a8_vec)", fn);
    return KQ_EUNSUPPORTED;
  }
  if (!dtype_ok(y_dtype)) { set_error("%s: unsupported output dtype %d", fn, y_dtype); return KQ_EUNSUPPORTED; }
  if (!y || stride_y < n) { set_error("%s: bad output (null or stride_y < n)", fn); return KQ_EINVAL; }
  if ((uintptr_t)y % dtype_size(y_dtype)) { set_error("%s: misaligned output pointer", fn); return KQ_EINVAL; }
  if (tokens * top_k > 0x7fffffffll) { set_error("%s: tokens * top_k does not fit 31 bits", fn); return KQ_ELIMIT; }
  cudaStream_t st = (cudaStream_t)stream;
  Q8Ptrs P = q8_ptrs(scratch, p.L, n);
  Q8Ptrs Pq = P;   // only the row-major codes and scales are read
  Pq.qsp = nullptr; Pq.xh = nullptr; Pq.s8h = nullptr; Pq.dT = nullptr; Pq.qsu = nullptr;
  rc = launch_quantize(x, x_dtype, tokens, k, stride_x, &Pq, nullptr, p.L.kpad, st);
  if (rc) return rc;
  return launch_moe(W, type, experts, n, k, P.ds, P.qs, p.L.kpad, tokens, top_k, ids, nslots, expert_ids, num_post_padded, block, y,
                    y_dtype, stride_y, st);
}

int kq_moe_a8_vec(const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* x, int x_dtype, int64_t tokens,
                  int64_t stride_x, const int32_t* topk_ids, int top_k, void* y, int y_dtype, int64_t stride_y, void* scratch,
                  size_t scratch_bytes, void* stream) {
  return moe_common("kq_moe_a8_vec", false, W, type, experts, n, k, x, x_dtype, tokens, stride_x, topk_ids, tokens * (int64_t)top_k,
                    nullptr, nullptr, top_k, y, y_dtype, stride_y, scratch, scratch_bytes, stream);
}

int kq_moe_a8(const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* x, int x_dtype, int64_t tokens,
              int64_t stride_x, const int32_t* sorted_token_ids, int64_t num_sorted, const int32_t* expert_ids,
              const int32_t* num_tokens_post_padded, int top_k, void* y, int y_dtype, int64_t stride_y, void* scratch,
              size_t scratch_bytes, void* stream) {
  return moe_common("kq_moe_a8", true, W, type, experts, n, k, x, x_dtype, tokens, stride_x, sorted_token_ids, num_sorted, expert_ids,
                    num_tokens_post_padded, top_k, y, y_dtype, stride_y, scratch, scratch_bytes, stream);
}

int kq_wait_arrival(const void* buf, size_t bytes, int dtype, int* status, void* stream) {
  t_err[0] = 0;
  if (!dtype_ok(dtype)) { set_error("kq_wait_arrival: unsupported dtype %d", dtype); return KQ_EUNSUPPORTED; }
  if (bytes == 0) return KQ_OK;
  if (!buf || !status || (uintptr_t)buf % 16 || bytes % 16) { set_error("kq_wait_arrival: null pointer, or buffer not 16-byte aligned and sized"); return KQ_EINVAL; }
  return launch_wait_arrival(buf, bytes, (int)dtype_size(dtype), status, (cudaStream_t)stream);
}

int kq_arrival_status(int* failed, int clear) {
  t_err[0] = 0;
  return arrival_status(failed, clear);
}

int kq_moe_block_size(int type) {
  int b, sz;
  return type_geometry(type, &b, &sz) ? KQ_MOE_BLOCK : 0;
}

int kq_debug_copy_window(uint64_t base, int64_t n, int64_t rowbytes, int64_t row_a, int64_t row_b, int64_t seg_off,
                         int64_t seg_len, int64_t* streamed_rows, uint64_t* bulk_start, uint64_t* bulk_bytes) {
  t_err[0] = 0;
  if (n <= 0 || rowbytes <= 0 || (rowbytes & 1) || (base & 15) || !streamed_rows || !bulk_start || !bulk_bytes) {
    set_error("kq_debug_copy_window: bad argument");
    return KQ_EINVAL;
  }
  const int64_t ns = stream_rows(n, rowbytes);
  *streamed_rows = ns;
  *bulk_start = 0; *bulk_bytes = 0;
  if (row_a < 0 || row_b <= row_a || row_b > ns) return KQ_OK;   // rows outside the streamed part: no window
  uintptr_t ga, ge;
  if (seg_len > 0) {   // one row segment (row_b is ignored)
    if (seg_off < 0 || seg_off + seg_len > rowbytes) { set_error("kq_debug_copy_window: segment outside the row"); return KQ_EINVAL; }
    ga = (uintptr_t)base + (uintptr_t)(row_a * rowbytes + seg_off);
    ge = ga + (uintptr_t)seg_len;
  } else {             // whole rows [row_a, row_b)
    ga = (uintptr_t)base + (uintptr_t)(row_a * rowbytes);
    ge = (uintptr_t)base + (uintptr_t)(row_b * rowbytes);
  }
  const CopyWindow w = copy_window(ga, ge);
  *bulk_start = (uint64_t)w.a0; *bulk_bytes = w.bulk;
  return KQ_OK;
}

int kq_set_option(const char* name, int value) {
  if (name && !strcmp(name, "gemv_impl")) { options().gemv_impl = value; return KQ_OK; }
  if (name && !strcmp(name, "half_fma")) { options().half_fma = value; return KQ_OK; }
  if (name && !strcmp(name, "tc_min_m")) { options().tc_min_m = value; return KQ_OK; }
  if (name && !strcmp(name, "gemm_min_m")) { options().gemm_min_m = value; return KQ_OK; }
  if (name && !strcmp(name, "tile_segments")) { options().tile_segments = value != 0; return KQ_OK; }
  if (name && !strcmp(name, "fuse_q8")) { options().fuse_q8 = value < 0 ? 0 : (value > 2 ? 2 : value); return KQ_OK; }
  if (name && !strcmp(name, "pdl")) { options().pdl = value < 0 ? 0 : value; return KQ_OK; }
  if (name && !strcmp(name, "kres")) { options().kres = value < 0 ? 0 : (value > 2 ? 2 : value); return KQ_OK; }
  if (name && !strcmp(name, "no_fused_gather")) { options().no_fused_gather = value != 0; return KQ_OK; }
  if (name && !strcmp(name, "gemm_wide")) { options().gemm_wide = value; return KQ_OK; }
  if (name && !strcmp(name, "gemm_small_m")) { options().gemm_small_m = value != 0; return KQ_OK; }
  if (name && !strcmp(name, "tile_two_stage")) { options().tile_two_stage = value != 0; return KQ_OK; }
  if (name && !strcmp(name, "moe_smem")) { options().moe_smem = value != 0; return KQ_OK; }
  if (name && !strcmp(name, "row_stage_kb")) { options().row_stage_kb = value < 4 ? 4 : (value > 96 ? 96 : value); return KQ_OK; }
  if (name && !strcmp(name, "umma")) { options().umma = value != 0; return KQ_OK; }
  if (name && !strcmp(name, "umma_min_m")) { options().umma_min_m = value; return KQ_OK; }
  if (name && !strcmp(name, "umma_box")) { options().umma_box = value != 0; return KQ_OK; }
  set_error("kq_set_option: unknown option");
  return KQ_EINVAL;
}

int kq_get_option(const char* name, int* value) {
  if (name && value && !strcmp(name, "gemv_impl")) { *value = options().gemv_impl; return KQ_OK; }
  if (name && value && !strcmp(name, "half_fma")) { *value = options().half_fma; return KQ_OK; }
  if (name && value && !strcmp(name, "tc_min_m")) { *value = options().tc_min_m; return KQ_OK; }
  if (name && value && !strcmp(name, "gemm_min_m")) { *value = options().gemm_min_m; return KQ_OK; }
  if (name && value && !strcmp(name, "tile_segments")) { *value = options().tile_segments; return KQ_OK; }
  if (name && value && !strcmp(name, "fuse_q8")) { *value = options().fuse_q8; return KQ_OK; }
  if (name && value && !strcmp(name, "pdl")) { *value = options().pdl; return KQ_OK; }
  if (name && value && !strcmp(name, "kres")) { *value = options().kres; return KQ_OK; }
  if (name && value && !strcmp(name, "no_fused_gather")) { *value = options().no_fused_gather; return KQ_OK; }
  if (name && value && !strcmp(name, "gemm_wide")) { *value = options().gemm_wide; return KQ_OK; }
  if (name && value && !strcmp(name, "gemm_small_m")) { *value = options().gemm_small_m; return KQ_OK; }
  if (name && value && !strcmp(name, "tile_two_stage")) { *value = options().tile_two_stage; return KQ_OK; }
  if (name && value && !strcmp(name, "moe_smem")) { *value = options().moe_smem; return KQ_OK; }
  if (name && value && !strcmp(name, "row_stage_kb")) { *value = options().row_stage_kb; return KQ_OK; }
  if (name && value && !strcmp(name, "umma")) { *value = options().umma; return KQ_OK; }
  if (name && value && !strcmp(name, "umma_min_m")) { *value = options().umma_min_m; return KQ_OK; }
  if (name && value && !strcmp(name, "umma_box")) { *value = options().umma_box; return KQ_OK; }
  if (name && value && !strcmp(name, "launch_count")) { *value = (int)(options().launches & 0x7fffffff); return KQ_OK; }
  set_error("kq_get_option: unknown option");
  return KQ_EINVAL;
}

}  // extern "C"
