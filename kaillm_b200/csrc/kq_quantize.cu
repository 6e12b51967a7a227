// q8_1 activation quantizer.
//
// Arithmetic of quantize_q8_1 in the reference (vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:32-69):
// per 32 consecutive activations d = amax/127 (IEEE fp32 division), q = roundf(x/d), and the fp32 sum
// of the raw values taken in xor-butterfly order 16,8,4,2,1; d and the sum are stored as fp16.
// Columns k..kpad-1 (kpad = ceil(k/512)*512) quantize as zeros.
//
// Output goes to the split layout the GEMV/GEMM kernels read (half2 ds[m][kpad/32], int8 qs[m][kpad])
// and/or to the reference's 36-byte block layout.
#include <cstring>
#include <type_traits>

#include "kq_common.cuh"

namespace kq {

// One 32-block of one token, one value per lane (the whole warp calls this): d = amax / 127, codes, the fp32 butterfly
// sum, and every table of the scratch layout.  tslot: index of (token tile, block, token in tile) in the transposed tables.
__device__ __forceinline__ void quantize_block(float xi, int64_t row, int b, int lane, int kpad, int64_t tslot, const Q8Ptrs& P,
                                               uint8_t* __restrict__ wire36) {
  const int nb = kpad >> 5;
  const int col = b * 32 + lane;
  float amax = fabsf(xi);
  float sum = xi;
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
    sum += __shfl_xor_sync(0xffffffffu, sum, mask);
  }
  const float d = __fdiv_rn(amax, 127.0f);
  const int8_t q = amax == 0.0f ? (int8_t)0 : (int8_t)roundf(__fdiv_rn(xi, d));
  if (P.qs) P.qs[row * kpad + col] = q;
  int8_t* unit = P.qsu ? P.qsu + ((row >> 4) * (kpad >> 8) + (b >> 3)) * (int64_t)KQ_UNIT_TABLE : nullptr;   // this pass's tables of the block's unit
  if (unit) unit[((((col & 255) >> 4) * 16) + (row & 15)) * 16 + (col & 15)] = q;
  if (P.xh) P.xh[row * kpad + col] = __float2half_rn(__half2float(__float2half_rn(d)) * (float)q);
  if (P.qsp) {
    int8_t* pp = P.qsp + (row * (kpad >> 6) + (col >> 6)) * 80;
    pp[col & 63] = q;
    if ((col & 63) < 16) pp[64 + (col & 63)] = 0;   // keep the padding defined
  }
  if (wire36) wire36[(row * nb + b) * 36 + 4 + lane] = (uint8_t)q;
  const __half dh = __float2half_rn(d), sh = __float2half_rn(sum);
  if (P.dT != nullptr) {
    int s16 = q;
#pragma unroll
    for (int mask = 8; mask > 0; mask >>= 1) s16 += __shfl_xor_sync(0xffffffffu, s16, mask);
    const int s16b = __shfl_xor_sync(0xffffffffu, s16, 16);
    if (lane == 0) {
      const float df = __half2float(dh);
      P.dT[tslot] = df;
      P.z32[tslot] = df * (float)(s16 + s16b);   // exact: 11-bit x 13-bit significands
      P.zs8[tslot] = __half2float(sh);
      const int64_t t16 = ((row >> 4) * 2 * nb + 2 * b) * 16 + (row & 15);
      P.z16[t16] = df * (float)s16;
      P.z16[t16 + 16] = df * (float)s16b;
      P.z32r[row * nb + b] = df * (float)(s16 + s16b);
      P.z16r[(row * nb + b) * 2] = df * (float)s16;
      P.z16r[(row * nb + b) * 2 + 1] = df * (float)s16b;
      if (unit) {
        float* ut = reinterpret_cast<float*>(unit + 4096) + (b & 7) * 16 + (row & 15);
        ut[0] = df; ut[128] = df * (float)(s16 + s16b); ut[256] = __half2float(sh);
        ut[384 + (b & 7) * 16] = df * (float)s16; ut[384 + (b & 7) * 16 + 16] = df * (float)s16b;   // [2 (b & 7) + half][16 tokens]
      }
    }
  }
  if (lane == 0) {
    const __half2 v = __halves2half2(dh, sh);
    if (P.ds) P.ds[row * nb + b] = v;
    if (P.xh) P.s8h[row * nb + b] = sh;
    if (wire36) *reinterpret_cast<__half2*>(wire36 + (row * nb + b) * 36) = v;
  }
}

// Activations that are the output of a sharded projection whose all-gather has no hand-shake (kq_mul_mat_prepared_gather
// with `wait_in_consumer`): the buffer was filled with the sentinel (all bits set, a NaN no conversion produces) before
// the ranks stored into it, so a value is its own arrival flag.  The load is repeated - bounded, about two seconds - until
// it returns something else; it goes to L2 (system scope), where the peers' stores land.
// Once a wait has run out (a peer is gone), g_arrival_failed makes every later poll on this GPU give up at once instead of
// after its own two seconds; kq_arrival_status reads and clears it.
constexpr long long KQ_ARRIVAL_WAIT = 1ll << 32;
__device__ int g_arrival_failed = 0;
template <typename T>
__device__ __forceinline__ T load_arrived(const T* p, int* status) {
  using Bits = typename std::conditional<sizeof(T) == 2, unsigned short, unsigned int>::type;
  const Bits sentinel = (Bits)~(Bits)0;
  const volatile Bits* q = reinterpret_cast<const volatile Bits*>(p);
  Bits v = *q;
  if (v == sentinel) {
    const long long t0 = clock64();
    do {
      __nanosleep(40);
      v = *q;
      if (*(volatile int*)&g_arrival_failed) break;
      if (clock64() - t0 > KQ_ARRIVAL_WAIT) { atomicExch(status, 40); atomicExch(&g_arrival_failed, 40); break; }
    } while (v == sentinel);
  }
  T out;
  memcpy(&out, &v, sizeof(T));
  return out;
}
// sixteen bytes of such a buffer at once (L2 load; re-read while any element still holds the sentinel)
template <typename T>
__device__ __forceinline__ uint4 load_vec_arrived(const uint4* p, int wait_arrival, int* status) {
  uint4 v = __ldcg(p);
  if (wait_arrival) {
    auto missing = [](const uint4& w) {
      if constexpr (sizeof(T) == 2) return (__vcmpeq2(w.x, 0xFFFFFFFFu) | __vcmpeq2(w.y, 0xFFFFFFFFu) | __vcmpeq2(w.z, 0xFFFFFFFFu) | __vcmpeq2(w.w, 0xFFFFFFFFu)) != 0u;
      else return w.x == 0xFFFFFFFFu || w.y == 0xFFFFFFFFu || w.z == 0xFFFFFFFFu || w.w == 0xFFFFFFFFu;
    };
    if (missing(v)) {
      const long long t0 = clock64();
      do {
        __nanosleep(40);
        v = __ldcg(p);
        if (*(volatile int*)&g_arrival_failed) break;
        if (clock64() - t0 > KQ_ARRIVAL_WAIT) { atomicExch(status, 40); atomicExch(&g_arrival_failed, 40); break; }
      } while (missing(v));
    }
  }
  return v;
}
template <typename T>
__device__ __forceinline__ float load_act(const T* p, int wait_arrival, int* status) {
  return to_f32<T>(wait_arrival ? load_arrived<T>(p, status) : *p);
}

// Padding tokens (m .. 16 * ceil(m / 16) - 1): zero scales in the unit tables (their codes may be anything)
__device__ __forceinline__ void zero_unit_tables(const Q8Ptrs& P, int64_t row, int b, int kpad) {
  if (!P.qsu) return;
  float* ut = reinterpret_cast<float*>(P.qsu + ((row >> 4) * (kpad >> 8) + (b >> 3)) * (int64_t)KQ_UNIT_TABLE + 4096) + (b & 7) * 16 + (row & 15);
  ut[0] = 0.f; ut[128] = 0.f; ut[256] = 0.f; ut[384 + (b & 7) * 16] = 0.f; ut[384 + (b & 7) * 16 + 16] = 0.f;
}

// One warp per (token, 32-block).  Tokens m..16*ceil(m/16)-1 only zero-fill the transposed scale tables.
template <typename T>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const T* __restrict__ x, int64_t stride_x, int k,
                                                            int kpad, int64_t m, int64_t mpad, Q8Ptrs P,
                                                            uint8_t* __restrict__ wire36, int wait_arrival) {
  pdl_trigger();   // a GEMV launched behind this kernel may set up and prefetch its weights meanwhile
  pdl_wait();      // the scratch this kernel rewrites may still be read by the launch before it
  const int lane = threadIdx.x & 31;
  const int nb = kpad >> 5;
  const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (P.cnt != nullptr && gthread < P.ncnt) P.cnt[gthread] = 0;   // split-K counters start at zero
  if (P.status != nullptr && gthread == 0) P.status[0] = 0;
  const int64_t blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // global 32-block index over padded tokens
  if (blk >= mpad * nb) return;
  const int64_t row = blk / nb;
  const int b = (int)(blk - row * nb);
  const int64_t tslot = ((row >> 4) * nb + b) * 16 + (row & 15);      // [token tile][block][token in tile]
  if (row >= m) {
    if (P.dT != nullptr && lane == 0) {
      P.dT[tslot] = 0.f; P.z32[tslot] = 0.f; P.zs8[tslot] = 0.f;
      const int64_t t16 = ((row >> 4) * 2 * nb + 2 * b) * 16 + (row & 15);
      P.z16[t16] = 0.f; P.z16[t16 + 16] = 0.f;
      zero_unit_tables(P, row, b, kpad);
    }
    return;
  }
  const int col = b * 32 + lane;
  const float xi = col < k ? load_act<T>(x + row * stride_x + col, wait_arrival, P.status) : 0.0f;
  quantize_block(xi, row, b, lane, kpad, tslot, P, wire36);
}

// ---------------------------------------------------------------------------------------------- fused producers
// The activation of a projection group is usually the output of a small elementwise or normalising kernel.  These
// producers compute that output and quantize it in one launch, with the same per-block arithmetic as above (the
// reference's production backend fuses the same two producers into its own activation format:
// vllm_gguf_plugin/native/kernels/kai_prepare_ext.cuh:1-10, quantization/native_fused.py:144-200):
//   MODE 1  RMSNorm:  a = T(T(x * rsqrt(mean(x^2) + eps)) * gamma), both roundings in the storage type T, the order of
//                     vLLM's rms_norm kernel; optionally also stored as a dense [m, k] tensor (y_norm)
//   MODE 2  SwiGLU:   a = T(silu(gate)) * up in T, gate = gu[:, 0:k], up = gu[:, k:2k] - vLLM's SiluAndMul
// Grid = (tokens padded to 16, chunks of 8 blocks): one warp per 32-block, as in the plain quantizer; every CTA of an
// RMSNorm row recomputes the row's sum of squares (k loads per CTA, from L2).  Tokens m..16*ceil(m/16)-1 only
// zero-fill the transposed scale tables.
template <typename T> __device__ __forceinline__ T mul_in_type(T a, T b);
template <> __device__ __forceinline__ float mul_in_type<float>(float a, float b) { return a * b; }
template <> __device__ __forceinline__ __half mul_in_type<__half>(__half a, __half b) { return __hmul(a, b); }
template <> __device__ __forceinline__ __nv_bfloat16 mul_in_type<__nv_bfloat16>(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmul(a, b); }

template <typename T, int MODE>
__global__ void __launch_bounds__(256) prepare_fused_kernel(const T* __restrict__ x, int64_t stride_x, int k, int kpad,
                                                            int64_t m, const T* __restrict__ gamma, float eps,
                                                            T* __restrict__ y_norm, Q8Ptrs P, int wait_arrival) {
  pdl_trigger();
  pdl_wait();      // the scratch this kernel rewrites, and x, may still be in use by the launch before it
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nb = kpad >> 5;
  const int64_t row = blockIdx.x;
  const int b = blockIdx.y * 8 + warp;                 // this warp's 32-block
  const int64_t gthread = ((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t i = gthread; i < P.ncnt; i += (int64_t)gridDim.x * gridDim.y * blockDim.x) P.cnt[i] = 0;
  if (gthread == 0) P.status[0] = 0;
  if (row >= m) {
    if (b < nb && lane == 0) {
      const int64_t tslot = ((row >> 4) * nb + b) * 16 + (row & 15);
      P.dT[tslot] = 0.f; P.z32[tslot] = 0.f; P.zs8[tslot] = 0.f;
      const int64_t t16 = ((row >> 4) * 2 * nb + 2 * b) * 16 + (row & 15);
      P.z16[t16] = 0.f; P.z16[t16 + 16] = 0.f;
      zero_unit_tables(P, row, b, kpad);
    }
    return;
  }
  const T* xr = x + row * stride_x;
  float inv = 1.0f;
  if constexpr (MODE == 1) {
    __shared__ float s_part[8];
    float ss = 0.f;
    constexpr int PER = 16 / (int)sizeof(T);   // elements per 16-byte load
    if ((k % PER) == 0 && ((uintptr_t)xr % 16) == 0) {
      for (int c = threadIdx.x * PER; c < k; c += blockDim.x * PER) {
        const uint4 v = load_vec_arrived<T>(reinterpret_cast<const uint4*>(xr + c), wait_arrival, P.status);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int i = 0; i < PER; ++i) { const float f = to_f32<T>(e[i]); ss = fmaf(f, f, ss); }
      }
    } else {
      for (int c = threadIdx.x; c < k; c += blockDim.x) { const float v = load_act<T>(xr + c, wait_arrival, P.status); ss = fmaf(v, v, ss); }
    }
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, mask);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += s_part[w];
    inv = rsqrtf(tot / (float)k + eps);
  }
  if (b < nb) {
    const int col = b * 32 + lane;
    float xi = 0.0f;
    if (col < k) {
      T a;
      if constexpr (MODE == 1) {
        a = mul_in_type<T>(from_f32<T>(load_act<T>(xr + col, wait_arrival, P.status) * inv), gamma[col]);
        if (y_norm != nullptr) y_norm[row * k + col] = a;
      } else {
        const float g = load_act<T>(xr + col, wait_arrival, P.status);
        a = mul_in_type<T>(from_f32<T>(g / (1.0f + expf(-g))), wait_arrival ? load_arrived<T>(xr + k + col, P.status) : xr[k + col]);
      }
      xi = to_f32<T>(a);
    }
    const int64_t tslot = ((row >> 4) * nb + b) * 16 + (row & 15);
    quantize_block(xi, row, b, lane, kpad, tslot, P, nullptr);
  }
}

template <int MODE>
static int launch_prepare_fused(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, const void* gamma,
                                float eps, void* y_norm, const Q8Ptrs& P, cudaStream_t st, int wait_arrival) {
  const int64_t mpad = (m + 15) / 16 * 16;
  const bool pdl = options().pdl != 0;
  const dim3 grid((unsigned)mpad, (unsigned)((P.kpad / 32 + 7) / 8));
  cudaError_t rc;
  switch (x_dtype) {
    case KQ_F32: rc = launch_pdl(prepare_fused_kernel<float, MODE>, grid, dim3(256), 0, st, pdl, (const float*)x, stride_x, (int)k, (int)P.kpad, m, (const float*)gamma, eps, (float*)y_norm, P, wait_arrival); break;
    case KQ_F16: rc = launch_pdl(prepare_fused_kernel<__half, MODE>, grid, dim3(256), 0, st, pdl, (const __half*)x, stride_x, (int)k, (int)P.kpad, m, (const __half*)gamma, eps, (__half*)y_norm, P, wait_arrival); break;
    case KQ_BF16: rc = launch_pdl(prepare_fused_kernel<__nv_bfloat16, MODE>, grid, dim3(256), 0, st, pdl, (const __nv_bfloat16*)x, stride_x, (int)k, (int)P.kpad, m, (const __nv_bfloat16*)gamma, eps, (__nv_bfloat16*)y_norm, P, wait_arrival); break;
    default: set_error("unsupported activation dtype %d", x_dtype); return KQ_EUNSUPPORTED;
  }
  KQ_CUDA_TRY(rc);
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

int launch_prepare_rmsnorm(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, const void* gamma, float eps,
                           void* y_norm, const Q8Ptrs& P, cudaStream_t st, int wait_arrival) {
  return launch_prepare_fused<1>(x, x_dtype, m, k, stride_x, gamma, eps, y_norm, P, st, wait_arrival);
}
int launch_prepare_swiglu(const void* gate_up, int x_dtype, int64_t m, int64_t k, int64_t stride_gu, const Q8Ptrs& P,
                          cudaStream_t st, int wait_arrival) {
  return launch_prepare_fused<2>(gate_up, x_dtype, m, k, stride_gu, nullptr, 0.f, nullptr, P, st, wait_arrival);
}

// Waits until no element of buf[0 .. n16 * 16 bytes) holds the arrival sentinel (all bits of an element set): the end of
// a chain of sentinel-polled gathers, before a consumer outside the library reads the buffer.
__global__ void __launch_bounds__(256) wait_arrival_kernel(const uint4* buf, size_t n16, int elem_bytes, int* status) {
  const size_t nthr = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += nthr) {
    const volatile uint32_t* q = reinterpret_cast<const volatile uint32_t*>(buf + i);
    const long long t0 = clock64();
    for (;;) {
      bool missing = false;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w = q[j];
        missing |= elem_bytes == 2 ? __vcmpeq2(w, 0xFFFFFFFFu) != 0u : w == 0xFFFFFFFFu;
      }
      if (!missing) break;
      __nanosleep(100);
      if (*(volatile int*)&g_arrival_failed) { atomicExch(status, 41); break; }
      if (clock64() - t0 > KQ_ARRIVAL_WAIT) { atomicExch(status, 41); atomicExch(&g_arrival_failed, 41); break; }
    }
  }
}

int launch_wait_arrival(const void* buf, size_t bytes, int elem_bytes, int* status, cudaStream_t st) {
  if (bytes == 0) return KQ_OK;
  const size_t n16 = bytes / 16;
  size_t blocks = (n16 + 255) / 256;
  if (blocks > 592) blocks = 592;
  wait_arrival_kernel<<<(unsigned)blocks, 256, 0, st>>>((const uint4*)buf, n16, elem_bytes, status);
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

// (failed != nullptr) copies the flag to the host - synchronises; clear != 0 zeroes it afterwards
int arrival_status(int* failed, int clear) {
  int v = 0;
  KQ_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_arrival_failed, sizeof(int)));
  if (failed) *failed = v;
  if (clear && v) { const int z = 0; KQ_CUDA_TRY(cudaMemcpyToSymbol(g_arrival_failed, &z, sizeof(int))); }
  return KQ_OK;
}

// GEMM-only flavour (large M): one LANE per (token, 32-block).  Writes only what the tcgen05 GEMM reads: the fp16
// activations d*q and the fp16 raw block sums.  Same values as quantize_q8_1_kernel: amax and the codes do not depend on
// the order, and the fp32 block sum is formed by the tree of that kernel's xor butterfly (pairs 16 apart, then 8, 4, 2, 1).
template <typename T>
__global__ void __launch_bounds__(256) quantize_xh_kernel(const T* __restrict__ x, int64_t stride_x, int k, int kpad,
                                                          int64_t m, Q8Ptrs P) {
  pdl_trigger();
  pdl_wait();
  const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (P.cnt != nullptr && gthread < P.ncnt) P.cnt[gthread] = 0;
  if (P.status != nullptr && gthread == 0) P.status[0] = 0;
  const int nbk = k >> 5, nb = kpad >> 5;
  if (gthread >= m * nbk) return;
  const int64_t row = gthread / nbk;
  const int b = (int)(gthread - row * nbk);
  const T* src = x + row * stride_x + (int64_t)b * 32;
  float v[32];
  if constexpr (sizeof(T) == 2) {
    uint32_t w[16];
    if (((uintptr_t)src & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 u = reinterpret_cast<const uint4*>(src)[i];
        w[4 * i] = u.x; w[4 * i + 1] = u.y; w[4 * i + 2] = u.z; w[4 * i + 3] = u.w;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const T lo = *reinterpret_cast<const T*>(reinterpret_cast<const uint16_t*>(&w[i]));
        const T hi = *reinterpret_cast<const T*>(reinterpret_cast<const uint16_t*>(&w[i]) + 1);
        v[2 * i] = to_f32<T>(lo); v[2 * i + 1] = to_f32<T>(hi);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = to_f32<T>(src[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = to_f32<T>(src[i]);
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float d = __fdiv_rn(amax, 127.0f);
  const float dh = __half2float(__float2half_rn(d));
  uint32_t out[16];
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float q0 = amax == 0.0f ? 0.f : (float)(int8_t)roundf(__fdiv_rn(v[i], d));
    const float q1 = amax == 0.0f ? 0.f : (float)(int8_t)roundf(__fdiv_rn(v[i + 1], d));
    const __half2 h = __halves2half2(__float2half_rn(dh * q0), __float2half_rn(dh * q1));
    out[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
#pragma unroll
    for (int i = 0; i < off; ++i) v[i] = v[i] + v[i + off];
  uint4* dst = reinterpret_cast<uint4*>(P.xh + row * kpad + (int64_t)b * 32);   // kpad is a multiple of 512: 16-byte aligned
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[i] = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
  P.s8h[row * nb + b] = __float2half_rn(v[0]);
}

int launch_quantize(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, const Q8Ptrs* Pp,
                    void* wire36, int64_t kpad, cudaStream_t st, int wait_arrival) {
  Q8Ptrs P;
  if (Pp) P = *Pp; else { P = Q8Ptrs(); P.ds = nullptr; P.qs = nullptr; P.qsp = nullptr; P.xh = nullptr; P.s8h = nullptr; P.dT = P.z32 = P.zs8 = P.z16 = P.z32r = P.z16r = P.part = nullptr; P.qsu = nullptr; P.cnt = P.status = nullptr; P.kpad = kpad; P.ncnt = 0; }
  const bool pdl_on = options().pdl != 0;
  if (P.xh && P.s8h && !P.qs && !P.qsp && !P.ds && !P.dT && !wire36 && (k % 32) == 0 && m > 0) {
    // only the GEMM's operands are wanted (large M): lane-per-block kernel
    int64_t gl = (m * (k / 32) + 255) / 256;
    if (gl * 256 < P.ncnt) gl = (P.ncnt + 255) / 256;
    cudaError_t rc2;
    switch (x_dtype) {
      case KQ_F32: rc2 = launch_pdl(quantize_xh_kernel<float>, dim3((unsigned)gl), dim3(256), 0, st, pdl_on, (const float*)x, stride_x, (int)k, (int)kpad, m, P); break;
      case KQ_F16: rc2 = launch_pdl(quantize_xh_kernel<__half>, dim3((unsigned)gl), dim3(256), 0, st, pdl_on, (const __half*)x, stride_x, (int)k, (int)kpad, m, P); break;
      case KQ_BF16: rc2 = launch_pdl(quantize_xh_kernel<__nv_bfloat16>, dim3((unsigned)gl), dim3(256), 0, st, pdl_on, (const __nv_bfloat16*)x, stride_x, (int)k, (int)kpad, m, P); break;
      default: set_error("unsupported activation dtype %d", x_dtype); return KQ_EUNSUPPORTED;
    }
    KQ_CUDA_TRY(rc2);
    options().launches += 1;
    KQ_CUDA_TRY(cudaGetLastError());
    return KQ_OK;
  }
  const int64_t mpad = Pp ? (m + 15) / 16 * 16 : m;
  const int64_t nblk = mpad * (kpad / 32);
  if (nblk == 0) return KQ_OK;
  int64_t gridl = (nblk + 7) / 8;
  if (gridl * 256 < P.ncnt) gridl = (P.ncnt + 255) / 256;
  const unsigned grid = (unsigned)gridl;
  const bool pdl = options().pdl != 0;
  cudaError_t lrc = cudaSuccess;
  switch (x_dtype) {
    case KQ_F32:
      lrc = launch_pdl(quantize_q8_1_kernel<float>, dim3(grid), dim3(256), 0, st, pdl, (const float*)x, stride_x, (int)k,
                       (int)kpad, m, mpad, P, (uint8_t*)wire36, wait_arrival);
      break;
    case KQ_F16:
      lrc = launch_pdl(quantize_q8_1_kernel<__half>, dim3(grid), dim3(256), 0, st, pdl, (const __half*)x, stride_x, (int)k,
                       (int)kpad, m, mpad, P, (uint8_t*)wire36, wait_arrival);
      break;
    case KQ_BF16:
      lrc = launch_pdl(quantize_q8_1_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, pdl, (const __nv_bfloat16*)x, stride_x, (int)k,
                       (int)kpad, m, mpad, P, (uint8_t*)wire36, wait_arrival);
      break;
    default:
      set_error("unsupported activation dtype %d", x_dtype);
      return KQ_EUNSUPPORTED;
  }
  KQ_CUDA_TRY(lrc);
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

}  // namespace kq
