// Mixture-of-experts GEMV/GEMM over expert-major GGUF weights W[E][n][row bytes]: every output row z of Y is one
// (token, expert) pair, y[z] = W[expert(z)] * q8_1(x[token(z)]).
//
//   vec    (ggml_moe_a8_vec, vllm_gguf_plugin/csrc/gguf/moe_vec.cuh:4-52, gguf_kernel.cu:395-530): z = token * top_k + j,
//          expert = topk_ids[z]; MMVQ arithmetic (vecdotq.cuh vec_dot_*_q8_1)
//   block  (ggml_moe_a8, csrc/gguf/moe.cuh:9-128, gguf_kernel.cu:292-393): the (token, expert) pairs arrive sorted by
//          expert in blocks of KQ_MOE_BLOCK slots (vLLM's moe_align_block_size with the size ggml_moe_get_block_size
//          returns); block b belongs to expert_ids[b], slot s holds z = sorted_token_ids[s] (z >= tokens * top_k: padding),
//          token = z / top_k; MMQ arithmetic.  A block's weights are decoded once for all of its slots.
//
// One warp per weight row: lanes take 32-weight sub-blocks round-robin, decode them to int8 words and form the exact
// integer dots with dp4a (the same arithmetic as the general GEMV kernel).  Experts outside [0, E) and padding slots are
// skipped, their output rows keep what the caller put there (the reference returns zeros for them).
#include "kq_common.cuh"

namespace kq {

namespace {

__device__ const uint16_t c_iq3s_codes_moe[512] = {
#include "kq_iq3s_codes.inc"
};

struct MoeParams {
  const uint8_t* W;
  int64_t rowbytes, expert_stride;   // bytes per row / per expert
  int n, nsb, experts;
  const __half2* ds;                 // activation scales [tokens][kpad/32]
  const int8_t* qs;                  // activation codes [tokens][kpad]
  int kpad, tokens, top_k;
  const int32_t* ids;                // vec: topk_ids [tokens * top_k]; block: sorted_token_ids
  const int32_t* expert_ids;         // block mode only
  const int32_t* num_post_padded;    // block mode only
  int64_t nslots;                    // tokens * top_k (vec) / entries of sorted_token_ids (block)
  void* y;
  int64_t stride_y;
};

template <int QT, int MT, bool MMQ, bool BLOCK, typename OutT>
__global__ void __launch_bounds__(128) moe_dp4a_kernel(const MoeParams p) {
  using F = Fmt<QT>;
  __shared__ uint32_t s_grid[QT == KQ_TYPE_IQ3_S ? 512 : 1];
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x) s_grid[i] = iq3s_expand(c_iq3s_codes_moe[i], KQ_IQ3S_TOP);
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= p.n) return;
  const int64_t total = (int64_t)p.tokens * p.top_k;
  // the slots of this CTA: their activation rows and output rows (-1: nothing to do)
  int tok[MT], dst[MT];
  int expert;
  if constexpr (BLOCK) {
    const int64_t s0 = (int64_t)blockIdx.y * MT;
    if (s0 > (int64_t)p.num_post_padded[0]) return;   // the reference's bound (moe.cuh:37)
    expert = p.expert_ids[blockIdx.y];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const int64_t s = s0 + t;
      const int z = s < p.nslots ? p.ids[s] : -1;
      const bool ok = z >= 0 && z < total;
      dst[t] = ok ? z : -1;
      tok[t] = ok ? z / p.top_k : 0;
    }
  } else {
    const int64_t z = blockIdx.y;
    expert = p.ids[z];
    dst[0] = (int)z;
    tok[0] = (int)(z / p.top_k);
  }
  if (expert < 0 || expert >= p.experts) return;
  const uint8_t* wrow = p.W + (size_t)expert * p.expert_stride + (size_t)row * p.rowbytes;
  const int nb8 = p.kpad >> 5;
  constexpr int NG = 32 / F::GROUP;

  float acc[MT];
#pragma unroll
  for (int t = 0; t < MT; ++t) acc[t] = 0.f;
  for (int sb = lane; sb < p.nsb; sb += 32) {
    SubBlock s;
    decode_subblock<QT>(wrow, sb, s_grid, s);
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      if (dst[t] >= 0) {
        const uint4* ap = reinterpret_cast<const uint4*>(p.qs + (size_t)tok[t] * p.kpad + (size_t)sb * 32);
        const uint4 u0 = ap[0], u1 = ap[1];
        const float2 dsf = __half22float2(p.ds[(size_t)tok[t] * nb8 + sb]);
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
      }
    }
  }
  OutT* y = reinterpret_cast<OutT*>(p.y);
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    float v = acc[t];
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) v += __shfl_xor_sync(0xffffffffu, v, mask);
    if (lane == 0 && dst[t] >= 0) y[(size_t)dst[t] * p.stride_y + row] = from_f32<OutT>(v);
  }
}

// The block's (vec mode: the pair's) activations in shared memory: a CTA of eight warps copies the q8_1 codes and scales of its
// slots once and then walks MOE_ROWS_PER_CTA rows of the expert (a warp takes MOE_RW rows at a time), so the activations
// are read from global memory once per 64 rows instead of once per row.  Same arithmetic, same order of additions per row
// as moe_dp4a_kernel (bit-identical results).  Measured on 32 experts x Q4_K 2816x2048, top-4: block op at 256 tokens
// 1005 -> 384 us (the reference's kernel: 581), vec op at 8 tokens 42 -> 38 us (reference: 63); four rows per warp were
// slower than two (128 registers).
constexpr int MOE_ROWS_PER_CTA = 64;
#ifndef MOE_RW
#define MOE_RW 2
#endif
template <int QT, int MT, bool MMQ, bool BLOCK, typename OutT>
__global__ void __launch_bounds__(256) moe_block_smem_kernel(const MoeParams p) {
  using F = Fmt<QT>;
  extern __shared__ __align__(16) uint8_t moe_smem[];
  __shared__ uint32_t s_grid[QT == KQ_TYPE_IQ3_S ? 512 : 1];
  const int nb8 = p.kpad >> 5;
  int8_t* sQ = reinterpret_cast<int8_t*>(moe_smem);                                    // [MT][kpad]
  __half2* sDS = reinterpret_cast<__half2*>(moe_smem + (size_t)MT * p.kpad);           // [MT][kpad / 32]
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x) s_grid[i] = iq3s_expand(c_iq3s_codes_moe[i], KQ_IQ3S_TOP);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t total = (int64_t)p.tokens * p.top_k;
  int tok[MT], dst[MT];
  int expert;
  if constexpr (BLOCK) {
    const int64_t s0 = (int64_t)blockIdx.y * MT;
    if (s0 > (int64_t)p.num_post_padded[0]) return;   // the reference's bound (moe.cuh:37)
    expert = p.expert_ids[blockIdx.y];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const int64_t s = s0 + t;
      const int z = s < p.nslots ? p.ids[s] : -1;
      const bool ok = z >= 0 && z < total;
      dst[t] = ok ? z : -1;
      tok[t] = ok ? z / p.top_k : 0;
    }
  } else {                                            // vec mode (MT = 1): the grid row is the (token, expert) pair
    const int64_t z = blockIdx.y;
    expert = p.ids[z];
    dst[0] = (int)z;
    tok[0] = (int)(z / p.top_k);
  }
  if (expert < 0 || expert >= p.experts) return;
  {
    const int vec_per_row = p.kpad >> 4;             // 16-byte pieces of a token's codes
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      if (dst[t] < 0) continue;
      const uint4* src = reinterpret_cast<const uint4*>(p.qs + (size_t)tok[t] * p.kpad);
      uint4* d4 = reinterpret_cast<uint4*>(sQ + (size_t)t * p.kpad);
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d4[i] = __ldg(src + i);
      for (int i = threadIdx.x; i < nb8; i += blockDim.x) sDS[(size_t)t * nb8 + i] = p.ds[(size_t)tok[t] * nb8 + i];
    }
  }
  __syncthreads();
  constexpr int NG = 32 / F::GROUP;
  OutT* y = reinterpret_cast<OutT*>(p.y);
  const int row_end = min(p.n, (int)(blockIdx.x + 1) * MOE_ROWS_PER_CTA);
  // a warp takes MOE_RW rows at a time: a slot's codes and scales are read from shared memory once for all of them
  constexpr int RW = MOE_RW;
  for (int row = blockIdx.x * MOE_ROWS_PER_CTA + RW * warp; row < row_end; row += 8 * RW) {
    const uint8_t* wrow0 = p.W + (size_t)expert * p.expert_stride + (size_t)row * p.rowbytes;
    float acc[RW][MT];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int r = 0; r < RW; ++r) acc[r][t] = 0.f;
    for (int sb = lane; sb < p.nsb; sb += 32) {
      SubBlock sw[RW];
#pragma unroll
      for (int r = 0; r < RW; ++r)   // rows past the end re-read the last row (their sums are not stored)
        decode_subblock<QT>(wrow0 + (size_t)(row + r < row_end ? r : 0) * p.rowbytes, sb, s_grid, sw[r]);
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (dst[t] >= 0) {
          const uint4* ap = reinterpret_cast<const uint4*>(sQ + (size_t)t * p.kpad + (size_t)sb * 32);
          const uint4 u0 = ap[0], u1 = ap[1];
          const float2 dsf = __half22float2(sDS[(size_t)t * nb8 + sb]);
          const uint32_t u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
          int S[2] = {0, 0};
          if constexpr (F::HAS_MIN && !RawSum<QT, MMQ>::value) {
#pragma unroll
            for (int i = 0; i < 8; ++i) S[(NG == 2) ? (i >> 2) : 0] = __dp4a(0x01010101, (int)u[i], S[(NG == 2) ? (i >> 2) : 0]);
          }
#pragma unroll
          for (int r = 0; r < RW; ++r) {
            const SubBlock& s = sw[r];
            int I[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int h = (NG == 2) ? (i >> 2) : 0;
              I[h] = __dp4a((int)s.v[i], (int)u[i], I[h]);
            }
            float c;
            if constexpr (HalfProd<QT>::value) {
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
            acc[r][t] += c;
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) {
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        float v = acc[r][t];
#pragma unroll
        for (int mask = 16; mask > 0; mask >>= 1) v += __shfl_xor_sync(0xffffffffu, v, mask);
        if (lane == 0 && dst[t] >= 0 && row + r < row_end) y[(size_t)dst[t] * p.stride_y + row + r] = from_f32<OutT>(v);
      }
    }
  }
}

template <int QT, bool MMQ, typename OutT>
int run_moe(const MoeParams& p, bool block, cudaStream_t st) {
  const unsigned gx = (unsigned)((p.n + 3) / 4);
  if (block) {
    const int64_t nblocks = (p.nslots + KQ_MOE_BLOCK - 1) / KQ_MOE_BLOCK;
    if (nblocks > 65535) { set_error("kq_moe_a8: more than 65535 blocks of sorted tokens"); return KQ_ELIMIT; }
    const size_t smem = (size_t)KQ_MOE_BLOCK * p.kpad + (size_t)KQ_MOE_BLOCK * (p.kpad >> 5) * 4;
    if (nblocks > 0 && smem <= 200 * 1024 && options().moe_smem) {
      auto kern = moe_block_smem_kernel<QT, KQ_MOE_BLOCK, MMQ, true, OutT>;
      static DeviceOnce attr_set;
      if (attr_set.first_time()) {
        KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set.done();
      }
      const unsigned gr = (unsigned)((p.n + MOE_ROWS_PER_CTA - 1) / MOE_ROWS_PER_CTA);
      kern<<<dim3(gr, (unsigned)nblocks), 256, smem, st>>>(p);
    } else if (nblocks > 0) {
      moe_dp4a_kernel<QT, KQ_MOE_BLOCK, MMQ, true, OutT><<<dim3(gx, (unsigned)nblocks), 128, 0, st>>>(p);
    }
  } else {
    if (p.nslots > 65535) { set_error("kq_moe_a8_vec: more than 65535 (token, expert) pairs"); return KQ_ELIMIT; }
    const size_t smem = (size_t)p.kpad + (size_t)(p.kpad >> 5) * 4;
    if (p.nslots > 0 && smem <= 200 * 1024 && options().moe_smem) {
      auto kern = moe_block_smem_kernel<QT, 1, MMQ, false, OutT>;
      static DeviceOnce attr_set;
      if (attr_set.first_time()) {
        KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set.done();
      }
      const unsigned gr = (unsigned)((p.n + MOE_ROWS_PER_CTA - 1) / MOE_ROWS_PER_CTA);
      kern<<<dim3(gr, (unsigned)p.nslots), 256, smem, st>>>(p);
    } else if (p.nslots > 0) {
      moe_dp4a_kernel<QT, 1, MMQ, false, OutT><<<dim3(gx, (unsigned)p.nslots), 128, 0, st>>>(p);
    }
  }
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT, bool MMQ>
int run_moe_out(const MoeParams& p, bool block, int y_dtype, cudaStream_t st) {
  switch (y_dtype) {
    case KQ_F32: return run_moe<QT, MMQ, float>(p, block, st);
    case KQ_F16: return run_moe<QT, MMQ, __half>(p, block, st);
    case KQ_BF16: return run_moe<QT, MMQ, __nv_bfloat16>(p, block, st);
  }
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace

// block = false: ids = topk_ids; block = true: ids = sorted_token_ids (MMQ arithmetic)
int launch_moe(const void* W, int type, int64_t experts, int64_t n, int64_t k, const void* ds, const void* qs, int64_t kpad,
               int64_t tokens, int top_k, const int32_t* ids, int64_t nslots, const int32_t* expert_ids,
               const int32_t* num_post_padded, bool block, void* y, int y_dtype, int64_t stride_y, cudaStream_t st) {
  int blk, bytes;
  if (!type_geometry(type, &blk, &bytes)) { set_error("unsupported GGML type %d", type); return KQ_EUNSUPPORTED; }
  MoeParams p;
  p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.expert_stride = p.rowbytes * n; p.n = (int)n; p.nsb = (int)(k / 32);
  p.experts = (int)experts; p.ds = (const __half2*)ds; p.qs = (const int8_t*)qs; p.kpad = (int)kpad; p.tokens = (int)tokens;
  p.top_k = top_k; p.ids = ids; p.expert_ids = expert_ids; p.num_post_padded = num_post_padded; p.nslots = nslots;
  p.y = y; p.stride_y = stride_y;
  const bool mmq = block;
#define KQ_MOE_CASE(T) case T: return run_moe_out<T, false>(p, block, y_dtype, st)
#define KQ_MOE_CASE2(T) case T: return mmq ? run_moe_out<T, true>(p, block, y_dtype, st) : run_moe_out<T, false>(p, block, y_dtype, st)
  switch (type) {
    KQ_MOE_CASE(KQ_TYPE_Q4_0); KQ_MOE_CASE(KQ_TYPE_Q8_0); KQ_MOE_CASE(KQ_TYPE_Q2_K); KQ_MOE_CASE(KQ_TYPE_Q6_K);
    KQ_MOE_CASE(KQ_TYPE_IQ3_S); KQ_MOE_CASE(KQ_TYPE_Q4_1); KQ_MOE_CASE(KQ_TYPE_Q5_1); KQ_MOE_CASE(KQ_TYPE_Q3_K);
    KQ_MOE_CASE(KQ_TYPE_IQ4_NL); KQ_MOE_CASE(KQ_TYPE_IQ4_XS);
    KQ_MOE_CASE2(KQ_TYPE_Q4_K); KQ_MOE_CASE2(KQ_TYPE_Q5_0); KQ_MOE_CASE2(KQ_TYPE_Q5_K);
  }
#undef KQ_MOE_CASE
#undef KQ_MOE_CASE2
  set_error("unsupported GGML type %d", type);
  return KQ_EUNSUPPORTED;
}

}  // namespace kq
