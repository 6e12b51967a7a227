// Decode GEMV, dp4a flavour: one warp per weight row, weights read once for up to MT tokens.
//
// Lanes take 32-weight sub-blocks of the row round-robin, decode them to int8 words
// (decode_subblock) and form the exact integer dots against the q8_1 activation codes with dp4a;
// the fp32 combine per sub-block follows the reference's vec_dot_* functions
// (vllm_gguf_plugin/csrc/gguf/vecdotq.cuh:46-66, 165-177, 204-230, 328-379, 447-465, 1649-1672; the other formats:
// 71-160 Q4_1/Q5_0/Q5_1, 269-326 Q3_K, 384-445 Q5_K, 1757-1811 IQ4_NL/IQ4_XS).
// Plain global loads, so any row stride / alignment the wire format allows is accepted; this kernel
// is the general path and the integer-dot export used by the tests.
#include "kq_common.cuh"

namespace kq {

__device__ const uint16_t c_iq3s_codes[512] = {
#include "kq_iq3s_codes.inc"
};

template <int QT, int MT, bool MMQ, typename OutT>
__global__ void __launch_bounds__(128)
gemv_dp4a_kernel(const uint8_t* __restrict__ W, int64_t rowbytes, int n, int nsb, const __half2* __restrict__ ds,
                 const int8_t* __restrict__ qs, int kpad, int m0, int mcount, OutT* __restrict__ y, int64_t stride_y,
                 int32_t* __restrict__ dbg_dots, int32_t* __restrict__ dbg_sums) {
  using F = Fmt<QT>;
  __shared__ uint32_t s_grid[QT == KQ_TYPE_IQ3_S ? 512 : 1];
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x) s_grid[i] = iq3s_expand(c_iq3s_codes[i], KQ_IQ3S_TOP);
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n) return;
  const uint8_t* wrow = W + (size_t)row * rowbytes;
  const int nb8 = kpad >> 5;
  constexpr int NG = 32 / F::GROUP;  // integer-dot groups per sub-block (1 or 2)

  float acc[MT];
#pragma unroll
  for (int t = 0; t < MT; ++t) acc[t] = 0.f;

  for (int sb = lane; sb < nsb; sb += 32) {
    SubBlock s;
    decode_subblock<QT>(wrow, sb, s_grid, s);
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      if (t < mcount) {
        const int tok = m0 + t;
        const uint4* ap = reinterpret_cast<const uint4*>(qs + (size_t)tok * kpad + (size_t)sb * 32);
        const uint4 u0 = ap[0], u1 = ap[1];
        const float2 dsf = __half22float2(ds[(size_t)tok * nb8 + sb]);
        const uint32_t u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        int I[2] = {0, 0}, S[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int h = (NG == 2) ? (i >> 2) : 0;
          I[h] = __dp4a((int)s.v[i], (int)u[i], I[h]);
          if (F::HAS_MIN) S[h] = __dp4a(0x01010101, (int)u[i], S[h]);
        }
        float c;
        if constexpr (HalfProd<QT>::value) {
          // d * d8 and m * s8 rounded to fp16 first, as the reference's __hmul2 does (wb holds -m)
          c = __half2float(__float2half_rn(s.wa[0] * dsf.x)) * (float)I[0] - __half2float(__float2half_rn(s.wb[0] * dsf.y));
        } else if constexpr (NG == 1) {
          c = s.wa[0] * (dsf.x * (float)I[0]);
          if constexpr (F::HAS_MIN) {
            const float z = RawSum<QT, MMQ>::value ? dsf.y : dsf.x * (float)S[0];
            c -= s.wb[0] * z;
          }
        } else {
          c = dsf.x * (s.wa[0] * (float)I[0] + s.wa[1] * (float)I[1]);
          if constexpr (F::HAS_MIN) c -= dsf.x * (s.wb[0] * (float)S[0] + s.wb[1] * (float)S[1]);
        }
        acc[t] += c;
        if (dbg_dots) {
          const size_t ng = (size_t)nsb * NG;
#pragma unroll
          for (int h = 0; h < NG; ++h) {
            dbg_dots[((size_t)tok * n + row) * ng + (size_t)sb * NG + h] = I[h];
            if (dbg_sums && row == 0) {
              int sv = S[h];
              if (!F::HAS_MIN) {
                sv = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (NG == 1 || (i >> 2) == h) sv = __dp4a(0x01010101, (int)u[i], sv);
              }
              dbg_sums[(size_t)tok * ng + (size_t)sb * NG + h] = sv;
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    float v = acc[t];
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) v += __shfl_xor_sync(0xffffffffu, v, mask);
    if (lane == 0 && t < mcount && y) y[(size_t)(m0 + t) * stride_y + row] = from_f32<OutT>(v);
  }
}

template <int QT, bool MMQ, typename OutT>
static int run_typed(const uint8_t* W, int64_t rowbytes, int64_t n, int64_t k, const void* ds, const void* qs,
                     int64_t kpad, int64_t m, void* y, int64_t stride_y, int32_t* dbg_dots, int32_t* dbg_sums,
                     cudaStream_t st) {
  const int nsb = (int)(k / 32);
  const unsigned grid = (unsigned)((n + 3) / 4);
  for (int64_t m0 = 0; m0 < m;) {
    const int64_t left = m - m0;
#define KQ_LAUNCH(MT_)                                                                                              \
  gemv_dp4a_kernel<QT, MT_, MMQ, OutT><<<grid, 128, 0, st>>>(W, rowbytes, (int)n, nsb, (const __half2*)ds,         \
                                                             (const int8_t*)qs, (int)kpad, (int)m0,                 \
                                                             (int)(left < MT_ ? left : MT_), (OutT*)y, stride_y,    \
                                                             dbg_dots, dbg_sums)
    if (left >= 8) { KQ_LAUNCH(8); m0 += 8; }
    else if (left > 4) { KQ_LAUNCH(8); m0 += left; }
    else if (left > 2) { KQ_LAUNCH(4); m0 += left; }
    else if (left == 2) { KQ_LAUNCH(2); m0 += 2; }
    else { KQ_LAUNCH(1); m0 += 1; }
#undef KQ_LAUNCH
    options().launches += 1;
  }
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT, bool MMQ>
static int run_out(const uint8_t* W, int64_t rowbytes, int64_t n, int64_t k, const void* ds, const void* qs,
                   int64_t kpad, int64_t m, void* y, int y_dtype, int64_t stride_y, int32_t* dd, int32_t* dsum,
                   cudaStream_t st) {
  switch (y_dtype) {
    case KQ_F32: return run_typed<QT, MMQ, float>(W, rowbytes, n, k, ds, qs, kpad, m, y, stride_y, dd, dsum, st);
    case KQ_F16: return run_typed<QT, MMQ, __half>(W, rowbytes, n, k, ds, qs, kpad, m, y, stride_y, dd, dsum, st);
    case KQ_BF16: return run_typed<QT, MMQ, __nv_bfloat16>(W, rowbytes, n, k, ds, qs, kpad, m, y, stride_y, dd, dsum, st);
    default: set_error("unsupported output dtype %d", y_dtype); return KQ_EUNSUPPORTED;
  }
}

int launch_gemv_dp4a(const void* W, int type, int64_t n, int64_t k, const void* ds, const void* qs, int64_t kpad,
                     int64_t m, void* y, int y_dtype, int64_t stride_y, bool mmq, int32_t* dd, int32_t* dsum,
                     cudaStream_t st) {
  int blk, bytes;
  if (!type_geometry(type, &blk, &bytes)) { set_error("unsupported GGML type %d", type); return KQ_EUNSUPPORTED; }
  const int64_t rb = k / blk * bytes;
  const uint8_t* w = (const uint8_t*)W;
  switch (type) {
    case KQ_TYPE_Q4_0: return run_out<KQ_TYPE_Q4_0, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q8_0: return run_out<KQ_TYPE_Q8_0, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q2_K: return run_out<KQ_TYPE_Q2_K, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q4_K:
      return mmq ? run_out<KQ_TYPE_Q4_K, true>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st)
                 : run_out<KQ_TYPE_Q4_K, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q6_K: return run_out<KQ_TYPE_Q6_K, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_IQ3_S: return run_out<KQ_TYPE_IQ3_S, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q4_1: return run_out<KQ_TYPE_Q4_1, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q5_0:
      return mmq ? run_out<KQ_TYPE_Q5_0, true>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st)
                 : run_out<KQ_TYPE_Q5_0, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q5_1: return run_out<KQ_TYPE_Q5_1, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q3_K: return run_out<KQ_TYPE_Q3_K, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_Q5_K:
      return mmq ? run_out<KQ_TYPE_Q5_K, true>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st)
                 : run_out<KQ_TYPE_Q5_K, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_IQ4_NL: return run_out<KQ_TYPE_IQ4_NL, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
    case KQ_TYPE_IQ4_XS: return run_out<KQ_TYPE_IQ4_XS, false>(w, rb, n, k, ds, qs, kpad, m, y, y_dtype, stride_y, dd, dsum, st);
  }
  return KQ_EUNSUPPORTED;
}

}  // namespace kq
