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

template <typename T>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const T* __restrict__ x, int64_t stride_x, int k,
                                                            int kpad, int64_t m, __half2* __restrict__ ds,
                                                            int8_t* __restrict__ qs, uint8_t* __restrict__ wire36) {
  const int lane = threadIdx.x & 31;
  const int nb = kpad >> 5;
  const int64_t blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // global 32-block index
  if (blk >= m * nb) return;
  const int64_t row = blk / nb;
  const int b = (int)(blk - row * nb);
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
  if (qs) qs[row * kpad + col] = q;
  if (wire36) wire36[blk * 36 + 4 + lane] = (uint8_t)q;
  if (lane == 0) {
    const __half2 v = __halves2half2(__float2half_rn(d), __float2half_rn(sum));
    if (ds) ds[blk] = v;
    if (wire36) *reinterpret_cast<__half2*>(wire36 + blk * 36) = v;
  }
}

int launch_quantize(const void* x, int x_dtype, int64_t m, int64_t k, int64_t stride_x, void* ds, void* qs,
                    void* wire36, int64_t kpad, cudaStream_t st) {
  const int64_t nblk = m * (kpad / 32);
  if (nblk == 0) return KQ_OK;
  const unsigned grid = (unsigned)((nblk + 7) / 8);
  switch (x_dtype) {
    case KQ_F32:
      quantize_q8_1_kernel<float><<<grid, 256, 0, st>>>((const float*)x, stride_x, (int)k, (int)kpad, m,
                                                       (__half2*)ds, (int8_t*)qs, (uint8_t*)wire36);
      break;
    case KQ_F16:
      quantize_q8_1_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, stride_x, (int)k, (int)kpad, m,
                                                        (__half2*)ds, (int8_t*)qs, (uint8_t*)wire36);
      break;
    case KQ_BF16:
      quantize_q8_1_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, stride_x, (int)k, (int)kpad,
                                                               m, (__half2*)ds, (int8_t*)qs, (uint8_t*)wire36);
      break;
    default:
      set_error("unsupported activation dtype %d", x_dtype);
      return KQ_EUNSUPPORTED;
  }
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

}  // namespace kq
