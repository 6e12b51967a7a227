// q8_1 activation quantizer.
//
// Arithmetic of quantize_q8_1 in the reference (vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:32-69):
// per 32 consecutive activations d = amax/127 (IEEE fp32 division), q = roundf(x/d), and the fp32 sum
// of the raw values taken in xor-butterfly order 16,8,4,2,1; d and the sum are stored as fp16.
// Columns k..kpad-1 (kpad = ceil(k/512)*512) quantize as zeros.
//
// Output goes to the split layout the GEMV/GEMM kernels read (half2 ds[m][kpad/32], int8 qs[m][kpad])
// and/or to the reference's 36-byte block layout.
#include "kq_common.cuh"

namespace kq {

// One warp per (token, 32-block).  Tokens m..16*ceil(m/16)-1 only zero-fill the transposed scale tables.
template <typename T>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const T* __restrict__ x, int64_t stride_x, int k,
                                                            int kpad, int64_t m, int64_t mpad, Q8Ptrs P,
                                                            uint8_t* __restrict__ wire36) {
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
    }
    return;
  }
  const int col = b * 32 + lane;
  const float xi = col < k ? to_f32<T>(x[row * stride_x + col]) : 0.0f;
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
    }
  }
  if (lane == 0) {
    const __half2 v = __halves2half2(dh, sh);
    if (P.ds) P.ds[row * nb + b] = v;
    if (P.xh) P.s8h[row * nb + b] = sh;
    if (wire36) *reinterpret_cast<__half2*>(wire36 + (row * nb + b) * 36) = v;
  }
}

int launch_quantize(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, const Q8Ptrs* Pp,
                    void* wire36, int64_t kpad, cudaStream_t st) {
  Q8Ptrs P;
  if (Pp) P = *Pp; else { P = Q8Ptrs(); P.ds = nullptr; P.qs = nullptr; P.qsp = nullptr; P.xh = nullptr; P.s8h = nullptr; P.dT = P.z32 = P.zs8 = P.z16 = P.z32r = P.z16r = P.part = nullptr; P.cnt = P.status = nullptr; P.kpad = kpad; P.ncnt = 0; }
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
                       (int)kpad, m, mpad, P, (uint8_t*)wire36);
      break;
    case KQ_F16:
      lrc = launch_pdl(quantize_q8_1_kernel<__half>, dim3(grid), dim3(256), 0, st, pdl, (const __half*)x, stride_x, (int)k,
                       (int)kpad, m, mpad, P, (uint8_t*)wire36);
      break;
    case KQ_BF16:
      lrc = launch_pdl(quantize_q8_1_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, pdl, (const __nv_bfloat16*)x, stride_x, (int)k,
                       (int)kpad, m, mpad, P, (uint8_t*)wire36);
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
