// ggml_dequantize: wire bytes -> dense half / bfloat16 / float.
//
// The reference's K-quant and legacy kernels form each weight in fp16 and only then convert to the
// output type (vllm_gguf_plugin/csrc/gguf/dequantize.cuh:3-16, 69-78, 101-121, 156-196, 232-256); IQ3_S is
// formed in fp32 (dequantize.cuh:334-353).  The same operation order is kept here so results are
// bit-identical; `fma` selects whether a dependent fp16 multiply-subtract pair is contracted into one
// fused operation, which the CUDA compiler is free to do to the reference's `__hsub(__hmul(a,b),c)`
// (fma = 0: two roundings; 1: the first product is fused; 2: Q2_K's second product is fused instead).
//
// One thread produces 8 consecutive weights (16 bytes of fp16 output), so a warp writes 512 contiguous bytes.
#include <type_traits>

#include "kq_common.cuh"

namespace kq {

__device__ const uint16_t c_iq3s_codes_dq[512] = {
#include "kq_iq3s_codes.inc"
};

template <typename OutT> __device__ __forceinline__ OutT half_to_out(__half v);
template <> __device__ __forceinline__ __half half_to_out<__half>(__half v) { return v; }
template <> __device__ __forceinline__ float half_to_out<float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ __nv_bfloat16 half_to_out<__nv_bfloat16>(__half v) {
  return __float2bfloat16_rn(__half2float(v));
}

__device__ __forceinline__ __half mul_sub(__half a, __half b, __half c, int fma) {
  // a*b - c : one rounding if contracted, two otherwise
  return fma ? __hfma(a, b, __hneg(c)) : __hsub_rn(__hmul_rn(a, b), c);
}

// ---- two weights per instruction (the fp16 arithmetic of the reference, bit for bit: every step below is one correctly
// rounded fp16 operation on exact inputs, as in the scalar formulas)
// bytes i and i+1 of w (i = 0 or 2) as the halves (1024 + byte): fp16 1024..1279 has an ulp of 1, so OR-ing a byte into
// the mantissa of 1024 is exact
__device__ __forceinline__ __half2 bytes_to_h2_plus1024(uint32_t w, int i) {
  const uint32_t v = __byte_perm(w, 0u, i == 0 ? 0x4140u : 0x4342u) | 0x64006400u;
  return *reinterpret_cast<const __half2*>(&v);
}
// four fp16 pairs -> 8 outputs, one 16-byte (fp16 / bf16) or two (fp32) stores
template <typename OutT>
__device__ __forceinline__ void store8(OutT* dst, const __half2 (&h)[4]) {
  if constexpr (sizeof(OutT) == 4) {
    float4 a, b;
    const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
    a = make_float4(f0.x, f0.y, f1.x, f1.y); b = make_float4(f2.x, f2.y, f3.x, f3.y);
    reinterpret_cast<float4*>(dst)[0] = a; reinterpret_cast<float4*>(dst)[1] = b;
  } else if constexpr (std::is_same<OutT, __half>::value) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
  } else {
    __nv_bfloat162 o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __float22bfloat162_rn(__half22float2(h[i]));
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
  }
}

struct RowGather {
  const int64_t* ids;   // nullptr: the blocks are taken in storage order
  int64_t k, rowbytes, nrows;
  int f32math;          // Q4_K / Q5_K / Q6_K: fp32 products as gguf-reader and the reference's embedding decoder form them
};

// eight consecutive weights starting at element e0
template <int QT, typename OutT>
__device__ __forceinline__ void dequantize8(const uint8_t* __restrict__ W, int64_t e0, OutT* __restrict__ out, int fma,
                                            const RowGather& g, const uint32_t* s_grid) {
  using F = Fmt<QT>;
  const uint8_t* b = W + (e0 / F::BLK) * F::BYTES;
  if (g.ids != nullptr) {
    // output row r is weight row ids[r] (an embedding lookup); a row index outside the tensor gives zeros
    const int64_t r = e0 / g.k, src = g.ids[r];
    if (src < 0 || src >= g.nrows) {
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      reinterpret_cast<uint4*>(out + e0)[0] = z;
      if constexpr (sizeof(OutT) == 4) reinterpret_cast<uint4*>(out + e0)[1] = z;
      return;
    }
    b = W + src * g.rowbytes + ((e0 - r * g.k) / F::BLK) * F::BYTES;
  }
  const int r0 = (int)(e0 % F::BLK);
  OutT res[8];
  if constexpr (QT == KQ_TYPE_Q4_0) {
    const __half d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b));
    // the thread's 8 weights are the low (r0 < 16) or the high nibbles of 8 consecutive bytes; (q - 8) * d two at a time
    const uint8_t* q8 = b + 2 + (r0 & 15);
    const int sh = r0 >= 16 ? 4 : 0;
    const uint32_t w0 = (ld_u16x2(q8) >> sh) & 0x0F0F0F0Fu, w1 = (ld_u16x2(q8 + 4) >> sh) & 0x0F0F0F0Fu;
    const __half2 k1032 = __floats2half2_rn(1032.0f, 1032.0f), d2 = __halves2half2(d, d);
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __hmul2_rn(__hsub2_rn(bytes_to_h2_plus1024(i < 2 ? w0 : w1, (i & 1) * 2), k1032), d2);
    store8<OutT>(out + e0, h);
    return;
  } else if constexpr (QT == KQ_TYPE_Q8_0) {
    const __half d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b));
    {   // int8 codes -> fp16 by the biased-byte trick: (code ^ 0x80) + 1024 - 1152 = code
      const uint32_t w0 = ld_u16x2(b + 2 + r0) ^ 0x80808080u, w1 = ld_u16x2(b + 6 + r0) ^ 0x80808080u;
      const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f), d2 = __halves2half2(d, d);
      __half2 h[4];
      h[0] = __hmul2_rn(__hsub2_rn(bytes_to_h2_plus1024(w0, 0), bias), d2);
      h[1] = __hmul2_rn(__hsub2_rn(bytes_to_h2_plus1024(w0, 2), bias), d2);
      h[2] = __hmul2_rn(__hsub2_rn(bytes_to_h2_plus1024(w1, 0), bias), d2);
      h[3] = __hmul2_rn(__hsub2_rn(bytes_to_h2_plus1024(w1, 2), bias), d2);
      store8<OutT>(out + e0, h);
      return;
    }
  } else if constexpr (QT == KQ_TYPE_Q2_K) {
    const __half dall = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 80));
    const __half dmin = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 82));
    const int n = r0 >> 7, j4 = (r0 >> 5) & 3, l0 = r0 & 31;
    const int s = b[8 * n + 2 * j4 + (l0 >> 4)];
    const __half mpart = __hmul_rn(dmin, __int2half_rn(s >> 4));
    {   // two weights at a time: half(sc * q) = half(sc) * half(q) exactly (the product is at most 45)
      const uint8_t* q8 = b + 16 + 32 * n + l0;
      const bool al4 = ((uintptr_t)q8 & 3) == 0;
      const uint32_t w0 = ((al4 ? ld_u32(q8) : ld_u16x2(q8)) >> (2 * j4)) & 0x03030303u;
      const uint32_t w1 = ((al4 ? ld_u32(q8 + 4) : ld_u16x2(q8 + 4)) >> (2 * j4)) & 0x03030303u;
      const __half2 k1024 = __floats2half2_rn(1024.0f, 1024.0f), d2 = __halves2half2(dall, dall), m2 = __halves2half2(mpart, mpart);
      const __half sch = __int2half_rn(s & 15), mh = __int2half_rn(s >> 4);
      const __half2 s2 = __halves2half2(sch, sch), ndmin2 = __halves2half2(__hneg(dmin), __hneg(dmin)), mh2 = __halves2half2(mh, mh);
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 xq = __hmul2_rn(s2, __hsub2_rn(bytes_to_h2_plus1024(i < 2 ? w0 : w1, (i & 1) * 2), k1024));
        h[i] = fma == 2 ? __hfma2(ndmin2, mh2, __hmul2_rn(d2, xq))
                        : (fma ? __hfma2(d2, xq, __hneg2(m2)) : __hsub2_rn(__hmul2_rn(d2, xq), m2));
      }
      store8<OutT>(out + e0, h);
      return;
    }
  } else if constexpr (QT == KQ_TYPE_Q4_K) {
    const __half dall = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b));
    const __half dmin = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 2));
    const int il = r0 >> 6, hi = (r0 >> 5) & 1, l0 = r0 & 31;
    const int jj = 2 * il + hi;
    const uint8_t* q = b + 4;
    int sc, mn;
    if (jj < 4) { sc = q[jj] & 63; mn = q[jj + 4] & 63; }
    else { sc = (q[jj + 4] & 15) | ((q[jj - 4] >> 6) << 4); mn = (q[jj + 4] >> 4) | ((q[jj] >> 6) << 4); }
    const __half d1 = __hmul_rn(dall, __int2half_rn(sc));
    const __half m1 = __hmul_rn(dmin, __int2half_rn(mn));
    if (!g.f32math) {   // d1 * q - m1, two weights at a time
      const uint8_t* q8 = b + 16 + 32 * il + l0;
      const bool al4 = ((uintptr_t)q8 & 3) == 0;       // the tensor may start on a 2-byte boundary only
      const uint32_t r0w = al4 ? ld_u32(q8) : ld_u16x2(q8), r1w = al4 ? ld_u32(q8 + 4) : ld_u16x2(q8 + 4);
      const uint32_t w0 = (r0w >> (4 * hi)) & 0x0F0F0F0Fu, w1 = (r1w >> (4 * hi)) & 0x0F0F0F0Fu;
      const __half2 k1024 = __floats2half2_rn(1024.0f, 1024.0f), d2 = __halves2half2(d1, d1), m2 = __halves2half2(m1, m1);
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 q = __hsub2_rn(bytes_to_h2_plus1024(i < 2 ? w0 : w1, (i & 1) * 2), k1024);
        h[i] = fma ? __hfma2(d2, q, __hneg2(m2)) : __hsub2_rn(__hmul2_rn(d2, q), m2);
      }
      store8<OutT>(out + e0, h);
      return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int byte = b[16 + 32 * il + l0 + j];
      const int qq = hi ? (byte >> 4) : (byte & 15);
      if (g.f32math)   // (d * sc) * q - dmin * m with every product and the difference rounded in fp32
        res[j] = from_f32<OutT>(__fsub_rn(__fmul_rn(__fmul_rn(__half2float(dall), (float)sc), (float)qq),
                                          __fmul_rn(__half2float(dmin), (float)mn)));
      else
        res[j] = half_to_out<OutT>(mul_sub(d1, __int2half_rn(qq), m1, fma));
    }
  } else if constexpr (QT == KQ_TYPE_Q6_K) {
    const __half d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 208));
    const int ip = r0 >> 7, q4 = (r0 >> 5) & 3, l0 = r0 & 31;
    const int sc = (int8_t)b[192 + 8 * ip + 2 * q4 + (l0 >> 4)];
    if (!g.f32math) {   // d * half(sc * (code - 32)): sc and code - 32 are exact in fp16, so half(sc) * half(code - 32) rounds once, like the conversion of the integer product
      const uint8_t* pl = b + 64 * ip + 32 * (q4 & 1) + l0;
      const uint8_t* ph = b + 128 + 32 * ip + l0;
      const uint32_t l0w = ld_u16x2(pl), l1w = ld_u16x2(pl + 4), h0w = ld_u16x2(ph), h1w = ld_u16x2(ph + 4);
      const int sh = q4 < 2 ? 0 : 4;
      const uint32_t c0 = ((l0w >> sh) & 0x0F0F0F0Fu) | (((h0w >> (2 * q4)) & 0x03030303u) << 4);
      const uint32_t c1 = ((l1w >> sh) & 0x0F0F0F0Fu) | (((h1w >> (2 * q4)) & 0x03030303u) << 4);
      const __half2 k1056 = __floats2half2_rn(1056.0f, 1056.0f), d2 = __halves2half2(d, d);
      const __half sch = __int2half_rn(sc);
      const __half2 s2 = __halves2half2(sch, sch);
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 q = __hsub2_rn(bytes_to_h2_plus1024(i < 2 ? c0 : c1, (i & 1) * 2), k1056);
        h[i] = __hmul2_rn(d2, __hmul2_rn(s2, q));
      }
      store8<OutT>(out + e0, h);
      return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int lo = b[64 * ip + 32 * (q4 & 1) + l0 + j];
      const int nib = (q4 < 2) ? (lo & 15) : (lo >> 4);
      const int hb = (b[128 + 32 * ip + l0 + j] >> (2 * q4)) & 3;
      const int code = (nib | (hb << 4)) - 32;
      if (g.f32math) res[j] = from_f32<OutT>(__fmul_rn(__fmul_rn(__half2float(d), (float)sc), (float)code));   // (d * sc) * q
      else res[j] = half_to_out<OutT>(__hmul_rn(d, __int2half_rn(sc * code)));
    }
  } else if constexpr (QT == KQ_TYPE_IQ3_S) {
    const float dh = ld_h(b);
    const int ib = r0 >> 5, il = (r0 >> 3) & 3;
    const uint32_t qh = b[66 + ib];
    const uint32_t i1 = b[2 + 8 * ib + 2 * il] | ((qh << (8 - 2 * il)) & 256u);
    const uint32_t i2 = b[2 + 8 * ib + 2 * il + 1] | ((qh << (7 - 2 * il)) & 256u);
    const uint32_t g1 = s_grid[i1], g2 = s_grid[i2];
    const uint32_t signs = b[74 + 4 * ib + il];
    const uint32_t s4 = (b[106 + (ib >> 1)] >> (4 * (ib & 1))) & 15u;
    const float d = __fmul_rn(__fmul_rn(dh, 0.5f + (float)s4), 0.5f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t gb = ((j < 4 ? g1 : g2) >> (8 * (j & 3))) & 0xFFu;
      const float mag = __fmul_rn(d, __uint_as_float(gb | 0x4B000000u) - 8388608.0f);   // (float)gb without the conversion pipe
      res[j] = from_f32<OutT>(__uint_as_float(__float_as_uint(mag) ^ (((signs >> j) & 1u) << 31)));
    }
  } else if constexpr (QT == KQ_TYPE_Q4_1 || QT == KQ_TYPE_Q5_1 || QT == KQ_TYPE_Q5_0) {
    // dequantize.cuh:18-67: codes as fp16, then (q - 16) * d for Q5_0, q * d + m for Q4_1 / Q5_1 (the multiply-add pair
    // is contracted like the multiply-subtract of the K-quants when `fma` is set)
    constexpr int HDR = QT == KQ_TYPE_Q5_0 ? 2 : 4;
    const __half d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b));
    const __half m = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 2));   // Q4_1 / Q5_1 only
    uint32_t qh = 0;
    if constexpr (QT != KQ_TYPE_Q4_1) qh = (uint32_t)b[HDR] | ((uint32_t)b[HDR + 1] << 8) | ((uint32_t)b[HDR + 2] << 16) | ((uint32_t)b[HDR + 3] << 24);
    const uint8_t* qs = b + HDR + (QT == KQ_TYPE_Q4_1 ? 0 : 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = r0 + j;
      int q = e < 16 ? (qs[e] & 15) : (qs[e - 16] >> 4);
      if constexpr (QT != KQ_TYPE_Q4_1) q |= (int)((qh >> e) & 1u) << 4;
      __half v;
      if constexpr (QT == KQ_TYPE_Q5_0) v = __hmul_rn(__hsub_rn(__int2half_rn(q), __float2half_rn(16.0f)), d);
      else v = fma ? __hfma(__int2half_rn(q), d, m) : __hadd_rn(__hmul_rn(__int2half_rn(q), d), m);
      res[j] = half_to_out<OutT>(v);
    }
  } else if constexpr (QT == KQ_TYPE_Q3_K) {             // dequantize.cuh:123-152
    const __half dall = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 108));
    const int n = r0 >> 7, jq = (r0 >> 5) & 3, l0 = r0 & 31;
    const int is = 8 * n + 2 * jq + (l0 >> 4);
    const uint8_t* sc = b + 96;
    int us;
    if (is < 4) us = (sc[is] & 15) | (((sc[is + 8] >> 0) & 3) << 4);
    else if (is < 8) us = (sc[is] & 15) | (((sc[is + 4] >> 2) & 3) << 4);
    else if (is < 12) us = (sc[is - 8] >> 4) | (((sc[is] >> 4) & 3) << 4);
    else us = (sc[is - 8] >> 4) | (((sc[is - 4] >> 6) & 3) << 4);
    const __half dl = __hmul_rn(dall, __int2half_rn(us - 32));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int l = l0 + j;
      const int q = ((b[32 + 32 * n + l] >> (2 * jq)) & 3) - (((b[l] >> (4 * n + jq)) & 1) ? 0 : 4);
      res[j] = half_to_out<OutT>(__hmul_rn(dl, __int2half_rn(q)));
    }
  } else if constexpr (QT == KQ_TYPE_Q5_K) {             // dequantize.cuh:198-230
    const __half dall = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b));
    const __half dmin = __ushort_as_half(*reinterpret_cast<const uint16_t*>(b + 2));
    const int il = r0 >> 6, hi = (r0 >> 5) & 1, l0 = r0 & 31;
    const int jj = 2 * il + hi;
    const uint8_t* q = b + 4;
    int sc, mn;
    if (jj < 4) { sc = q[jj] & 63; mn = q[jj + 4] & 63; }
    else { sc = (q[jj + 4] & 15) | ((q[jj - 4] >> 6) << 4); mn = (q[jj + 4] >> 4) | ((q[jj] >> 6) << 4); }
    const __half d1 = __hmul_rn(dall, __int2half_rn(sc));
    const __half m1 = __hmul_rn(dmin, __int2half_rn(mn));
    if (!g.f32math) {   // as Q4_K, with the fifth bit of each code taken from qh
      const uint8_t* q8 = b + 48 + 32 * il + l0;
      const uint8_t* qh8 = b + 16 + l0;
      const bool al4 = ((uintptr_t)q8 & 3) == 0;
      const uint32_t r0w = al4 ? ld_u32(q8) : ld_u16x2(q8), r1w = al4 ? ld_u32(q8 + 4) : ld_u16x2(q8 + 4);
      const uint32_t h0w = al4 ? ld_u32(qh8) : ld_u16x2(qh8), h1w = al4 ? ld_u32(qh8 + 4) : ld_u16x2(qh8 + 4);
      const uint32_t w0 = ((r0w >> (4 * hi)) & 0x0F0F0F0Fu) | (((h0w >> jj) & 0x01010101u) << 4);
      const uint32_t w1 = ((r1w >> (4 * hi)) & 0x0F0F0F0Fu) | (((h1w >> jj) & 0x01010101u) << 4);
      const __half2 k1024 = __floats2half2_rn(1024.0f, 1024.0f), d2 = __halves2half2(d1, d1), m2 = __halves2half2(m1, m1);
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 q = __hsub2_rn(bytes_to_h2_plus1024(i < 2 ? w0 : w1, (i & 1) * 2), k1024);
        h[i] = fma ? __hfma2(d2, q, __hneg2(m2)) : __hsub2_rn(__hmul2_rn(d2, q), m2);
      }
      store8<OutT>(out + e0, h);
      return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int byte = b[48 + 32 * il + l0 + j];
      const int qq = (hi ? (byte >> 4) : (byte & 15)) + (((b[16 + l0 + j] >> jj) & 1) ? 16 : 0);
      if (g.f32math)
        res[j] = from_f32<OutT>(__fsub_rn(__fmul_rn(__fmul_rn(__half2float(dall), (float)sc), (float)qq),
                                          __fmul_rn(__half2float(dmin), (float)mn)));
      else
        res[j] = half_to_out<OutT>(mul_sub(d1, __int2half_rn(qq), m1, fma));
    }
  } else if constexpr (QT == KQ_TYPE_IQ4_NL || QT == KQ_TYPE_IQ4_XS) {   // dequantize.cuh:401-437: fp32 d * code value
    float d = ld_h(b);
    const uint8_t* qs;
    int e0b;                                             // position inside the 32-weight sub-block
    if constexpr (QT == KQ_TYPE_IQ4_NL) { qs = b + 2; e0b = r0; }
    else {
      const int ib = r0 >> 5;
      const uint32_t sh = *reinterpret_cast<const uint16_t*>(b + 2);
      const int ls = (int)(((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15u) | (((sh >> (2 * ib)) & 3u) << 4));
      d = __fmul_rn(d, (float)(ls - 32));
      qs = b + 8 + 16 * ib; e0b = r0 & 31;
    }
    // the thread's 8 weights are the low (e0b < 16) or the high nibbles of 8 consecutive bytes; the code values come from
    // two byte permutes per word (iq4nl_lookup), the int -> float conversion from the magic exponent
    const int sh4 = e0b >= 16 ? 4 : 0;
    const uint8_t* q8 = qs + (e0b & 15);
    uint32_t w[2];
    if constexpr (QT == KQ_TYPE_IQ4_NL) { w[0] = ld_u16x2(q8); w[1] = ld_u16x2(q8 + 4); }
    else { w[0] = ld_u32(q8); w[1] = ld_u32(q8 + 4); }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t kv4 = iq4nl_lookup((w[h] >> sh4) & 0x0F0F0F0Fu);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kv = (int)(int8_t)((kv4 >> (8 * i)) & 0xFFu);
        const float kf = __int_as_float(kv + 0x4B400000) - 12582912.0f;
        res[4 * h + i] = from_f32<OutT>(__fmul_rn(d, kf));
      }
    }
  }
  // 8 outputs = 16 (half/bf16) or 32 (float) contiguous, aligned bytes (Q4_0, Q8_0 and Q2_K have stored theirs already)
  if constexpr (QT != KQ_TYPE_Q4_0 && QT != KQ_TYPE_Q8_0 && QT != KQ_TYPE_Q2_K) {
    if constexpr (sizeof(OutT) == 2) {
      *reinterpret_cast<uint4*>(out + e0) = *reinterpret_cast<const uint4*>(res);
    } else {
      reinterpret_cast<uint4*>(out + e0)[0] = reinterpret_cast<const uint4*>(res)[0];
      reinterpret_cast<uint4*>(out + e0)[1] = reinterpret_cast<const uint4*>(res)[1];
    }
  }
}

// Grid-stride over chunks of eight weights (the launcher decides how many chunks a thread walks).
template <int QT, typename OutT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ W, int64_t count,
                                                         OutT* __restrict__ out, int fma, RowGather g) {
  // IQ3_S: the expanded codebook in shared memory (lanes look up different entries: the constant cache would serialise them)
  __shared__ uint32_t s_grid[QT == KQ_TYPE_IQ3_S ? 512 : 1];
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x) s_grid[i] = iq3s_expand(c_iq3s_codes_dq[i], KQ_IQ3S_TOP);
    __syncthreads();
  }
  const int64_t step = (int64_t)gridDim.x * blockDim.x * 8;
  for (int64_t e0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; e0 < count; e0 += step)
    dequantize8<QT, OutT>(W, e0, out, fma, g, s_grid);
}

template <int QT>
static int run(const void* W, int64_t count, void* out, int out_dtype, int fma, cudaStream_t st, const RowGather& g) {
  const int64_t threads = count / 8;
  int64_t blocks = (threads + 255) / 256;
  // IQ3_S fills its codebook once per CTA: few CTAs that walk many chunks; the other formats run best with one chunk per thread
  const int64_t cap = QT == KQ_TYPE_IQ3_S ? (int64_t)sm_count() * 16 : (int64_t)0x7fffffff;
  if (blocks > cap) blocks = cap;
  const unsigned grid = (unsigned)blocks;
  if (grid == 0) return KQ_OK;
  switch (out_dtype) {
    case KQ_F16: dequantize_kernel<QT, __half><<<grid, 256, 0, st>>>((const uint8_t*)W, count, (__half*)out, fma, g); break;
    case KQ_BF16: dequantize_kernel<QT, __nv_bfloat16><<<grid, 256, 0, st>>>((const uint8_t*)W, count, (__nv_bfloat16*)out, fma, g); break;
    case KQ_F32: dequantize_kernel<QT, float><<<grid, 256, 0, st>>>((const uint8_t*)W, count, (float*)out, fma, g); break;
    default: set_error("unsupported output dtype %d", out_dtype); return KQ_EUNSUPPORTED;
  }
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

int launch_dequantize(const void* W, int type, int64_t count, void* out, int out_dtype, cudaStream_t st, const int64_t* ids,
                      int64_t k, int64_t nrows, int f32math) {
  const int fma = options().half_fma;
  RowGather g;
  g.ids = ids; g.k = k; g.nrows = nrows; g.rowbytes = 0; g.f32math = f32math;
  if (ids) {
    int blk, bytes;
    if (!type_geometry(type, &blk, &bytes)) { set_error("unsupported GGML type %d", type); return KQ_EUNSUPPORTED; }
    g.rowbytes = k / blk * bytes;
  }
  switch (type) {
    case KQ_TYPE_Q4_0: return run<KQ_TYPE_Q4_0>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q8_0: return run<KQ_TYPE_Q8_0>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q2_K: return run<KQ_TYPE_Q2_K>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q4_K: return run<KQ_TYPE_Q4_K>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q6_K: return run<KQ_TYPE_Q6_K>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_IQ3_S: return run<KQ_TYPE_IQ3_S>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q4_1: return run<KQ_TYPE_Q4_1>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q5_0: return run<KQ_TYPE_Q5_0>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q5_1: return run<KQ_TYPE_Q5_1>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q3_K: return run<KQ_TYPE_Q3_K>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_Q5_K: return run<KQ_TYPE_Q5_K>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_IQ4_NL: return run<KQ_TYPE_IQ4_NL>(W, count, out, out_dtype, fma, st, g);
    case KQ_TYPE_IQ4_XS: return run<KQ_TYPE_IQ4_XS>(W, count, out, out_dtype, fma, st, g);
  }
  set_error("unsupported GGML type %d", type);
  return KQ_EUNSUPPORTED;
}

}  // namespace kq
