// Decode GEMV, small token counts: the row-streaming dp4a kernel (gemv_rows_kernel, described above its
// definition) and the dispatch over the decode kernels (launch_gemv_mma, bottom of the file).  Calls of 3..80 tokens
// go to the shared-stage int8 mma kernel of kq_gemv_tile.cu in passes of up to 16 tokens.
//
// The integer dots are exact; the fp32 combine follows the reference's vec_dot functions
// (vllm_gguf_plugin/csrc/gguf/vecdotq.cuh:46-66 Q4_0, 165-177 Q8_0, 204-263 Q2_K, 328-379 Q4_K, 447-491 Q6_K,
// 1649-1672 IQ3_S).
//
// Every wait is bounded: after ~2^27 clocks the waiter raises a CTA-wide abort flag and a status word in global
// memory, every warp leaves its loop, and the producer waits (again bounded) for the copies it has in flight
// before the CTA exits.
#include "kq_common.cuh"

namespace kq {

namespace {

constexpr long long WAIT_LIMIT = 1ll << 27;   // ~70 ms at 1.9 GHz; a healthy wait lasts microseconds
constexpr int SMEM_HEADER = 1024;
constexpr int MAX_STAGES = 32;

__device__ const uint16_t c_iq3s_codes_s[512] = {
#include "kq_iq3s_codes.inc"
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait; false = gave up (abort flag raised by this or another waiter)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT) { *abort_flag = 1; return false; }
  }
  return true;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------- row-streaming dp4a kernel
// Small M (1..8 tokens per pass).  A CTA owns a contiguous range of weight rows, so the split over the 148 SMs is
// balanced to one row and needs no split-K.  The producer fetches R whole consecutive rows per stage with ONE
// bulk copy (the copy engine handles of the order of ten million requests per second and SM, so requests must
// be >= ~5 KB to keep up with HBM; row segments of a K-split are far too small).  Row i of the CTA belongs to
// consumer warp i % 16; its 32 lanes take the row's 32-weight sub-blocks round-robin, decode each once and dot
// it against the MT tokens, and one butterfly at the end of the row forms the sum.  Warps only meet at the
// stage barriers: a stage is released when the warps owning its R rows have each arrived.
struct RowParams {
  const uint8_t* W;
  int64_t rowbytes;
  int n, nsb;               // rows, 32-weight sub-blocks per row
  int rows_per_stage, stages, stage_bytes;
  int a_stride, a_bytes, d_bytes, z_bytes;
  const int8_t* qs;
  const int8_t* qsp;        // padded codes [m][kpad/64][80]: 64 codes + 16 bytes of padding (pair mode)
  const __half2* ds;        // [m][kpad/32] {d, raw block sum}
  const float* zr;          // [m][kpad/32 * zpb] token-major min-term table (zmode 2, 3) or nullptr
  int zmode;                // min term: 0 none, 1 raw block sum from ds, 2 zr[b], 3 zr[2b], zr[2b+1]
  int zpb, kpad, nb32tot, klen;
  int m0, mcount;
  int prefetch;             // ring stages issued before waiting for the previous kernel
  const void* x;            // non-null: raw activations; the consumer warps quantize them into shared memory themselves
  int x_dtype;
  int64_t stride_x;
  void* y;
  int64_t stride_y;
  int* status;
};

constexpr int ROW_WARPS = 16;
constexpr int ROW_THREADS = (ROW_WARPS + 1) * 32;

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // unsigned bytes x signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// q8_1 quantization of the CTA's activations straight into shared memory (1-2 tokens), one LANE per 32-block.
// Bit-identical to quantize_q8_1_kernel, which gives a block to a warp: |x| max and the integer code sums do not
// depend on the order; the fp32 block sum is formed by the same tree as that kernel's xor butterfly (pairs 16 apart,
// then 8, 4, 2, 1: fp addition is commutative, so every lane of the butterfly holds this tree's value); d = amax/127
// and roundf(x/d) are the same IEEE operations.  Written in the layouts the consumers read; runs while the first
// weight stages are in flight.
template <bool PAIR>
__device__ __forceinline__ void quantize_rows_smem(const RowParams& p, uint8_t* sA, __half2* sDS, float* sZ, int warp,
                                                   int lane, int ntok) {
  const int nb = p.klen >> 5;
  const int esize = p.x_dtype == KQ_F32 ? 4 : 2;
  for (int idx = warp * 32 + lane; idx < ntok * nb; idx += ROW_WARPS * 32) {   // (token, block) pairs over all 512 lanes
    const int t = idx / nb, b = idx - t * nb;
    const uint8_t* xrow = reinterpret_cast<const uint8_t*>(p.x) + (size_t)(p.m0 + t) * p.stride_x * esize;
    {
      float v[32];
      const uint8_t* src = xrow + (size_t)b * 32 * esize;
      if (p.x_dtype == KQ_F32) {
        if (((uintptr_t)src & 15) == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 f = reinterpret_cast<const float4*>(src)[i];
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = reinterpret_cast<const float*>(src)[i];
        }
      } else {
        uint32_t w[16];
        if (((uintptr_t)src & 15) == 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 u = reinterpret_cast<const uint4*>(src)[i];
            w[4 * i] = u.x; w[4 * i + 1] = u.y; w[4 * i + 2] = u.z; w[4 * i + 3] = u.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = (uint32_t)reinterpret_cast<const uint16_t*>(src)[2 * i] | ((uint32_t)reinterpret_cast<const uint16_t*>(src)[2 * i + 1] << 16);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (p.x_dtype == KQ_BF16) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
          } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
          }
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
      const float d = __fdiv_rn(amax, 127.0f);
      uint32_t codes[8];
      int s16 = 0, s16b = 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int q = amax == 0.0f ? 0 : (int)(int8_t)roundf(__fdiv_rn(v[i], d));
        if (i < 16) s16 += q; else s16b += q;
        if ((i & 3) == 0) codes[i >> 2] = 0;
        codes[i >> 2] |= (uint32_t)(q & 0xFF) << (8 * (i & 3));
      }
      // block sum: the butterfly's tree
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int i = 0; i < off; ++i) v[i] = v[i] + v[i + off];
      const float sum = v[0];
      uint8_t* dst;
      if constexpr (PAIR) {
        uint8_t* grp = sA + (size_t)t * p.a_stride + (b >> 1) * 80;
        dst = grp + (b & 1) * 32;
        if ((b & 1) == 0) *reinterpret_cast<uint4*>(grp + 64) = make_uint4(0u, 0u, 0u, 0u);   // keep the padding defined
      } else {
        dst = sA + (size_t)t * p.a_stride + b * 32;
      }
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
      const __half dh = __float2half_rn(d), sh = __float2half_rn(sum);
      sDS[(size_t)t * p.nb32tot + b] = __halves2half2(dh, sh);
      const float df = __half2float(dh);
      if (p.zmode == 2) sZ[(size_t)t * p.nb32tot + b] = df * (float)(s16 + s16b);
      if (p.zmode == 3) {
        sZ[((size_t)t * p.nb32tot + b) * 2] = df * (float)s16;
        sZ[((size_t)t * p.nb32tot + b) * 2 + 1] = df * (float)s16b;
      }
    }
  }
}

// PAIR (Q4_K): a warp takes two rows at a time; lane = (row of the pair, super-block offset 0..3, quarter il 0..3)
// and handles one 32-byte run of nibbles = the two 32-weight sub-blocks 2il (low nibbles) and 2il+1 (high
// nibbles) of its super-block with 16-byte shared-memory loads.  The activation codes come from the padded
// layout (80 bytes per 64 codes) so that the eight lanes of a load phase hit eight different bank groups.
template <int QT, int MT, bool PAIR, typename OutT>
__global__ void __launch_bounds__(ROW_THREADS, 1) gemv_rows_kernel(const RowParams p) {
  using F = Fmt<QT>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + SMEM_HEADER - 8);
  volatile int* s_issued = reinterpret_cast<volatile int*>(smem + SMEM_HEADER - 16);
  uint32_t* s_grid = reinterpret_cast<uint32_t*>(smem + SMEM_HEADER);
  uint8_t* sA = smem + SMEM_HEADER + (QT == KQ_TYPE_IQ3_S ? 2048 : 0);
  __half2* sDS = reinterpret_cast<__half2*>(sA + p.a_bytes);                              // [MT][nb32tot]
  float* sZ = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sDS) + p.d_bytes);      // [MT][nb32tot*zpb]
  uint8_t* ring = reinterpret_cast<uint8_t*>(sZ) + p.z_bytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages, R = p.rows_per_stage;
  const int r0 = (int)((int64_t)blockIdx.x * p.n / gridDim.x), r1 = (int)((int64_t)(blockIdx.x + 1) * p.n / gridDim.x);
  pdl_trigger();
  if (r0 >= r1) return;
  const int nstages = (r1 - r0 + R - 1) / R;
  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + MAX_STAGES), bar_act = smem_u32(bars + 2 * MAX_STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, PAIR ? R / 2 : R); }
    mbar_init(bar_act, 1);
    *s_abort = 0;
    *s_issued = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += ROW_THREADS) s_grid[i] = iq3s_expand(c_iq3s_codes_s[i], KQ_IQ3S_TOP);
  }
  __syncthreads();

  if (warp == ROW_WARPS) {
    // ------------------------------------------------------------------ producer (one lane is enough)
    if (lane == 0) {
      auto issue_stage = [&](int q) {
        const int slot = q % S;
        const int ra = r0 + q * R;
        const int rb = (ra + R) < r1 ? (ra + R) : r1;
        // whole rows [ra, rb): one bulk copy (the host passes only row counts whose byte size is a multiple of 16,
        // so the rounded window stays inside the tensor).  This lane's loop is the request rate of the SM: a request
        // costs it ~0.25 us whatever its size, so stages are sized well above 16 KB (option row_stage_kb) and nothing
        // else sits in the loop (splitting a stage among several lanes made it slower)
        const CopyWindow cw = copy_window((uintptr_t)(p.W + (size_t)ra * p.rowbytes), (uintptr_t)(p.W + (size_t)rb * p.rowbytes));
        mbar_expect_tx(bar_full + 8 * slot, cw.bulk);
        bulk_g2s(smem_u32(ring + (size_t)slot * p.stage_bytes), (const void*)cw.a0, cw.bulk, bar_full + 8 * slot);
        __threadfence_block();
        *s_issued = q + 1;
      };
      // the weights do not depend on the previous kernel: fill the ring first, then wait for it
      int q = 0;
      for (; q < nstages && q < p.prefetch; ++q) issue_stage(q);
      pdl_wait();
      const int ntok = p.x != nullptr ? 0 : (p.mcount < MT ? p.mcount : MT);   // fused: the consumers quantize x themselves
      const uint32_t dsb = (uint32_t)p.nb32tot * 4u, zb = (uint32_t)p.nb32tot * p.zpb * 4u;   // multiples of 64 bytes
      const uint32_t alen = PAIR ? (uint32_t)(p.klen / 64) * 80u : (uint32_t)p.klen;
      uint32_t total = (uint32_t)ntok * (alen + dsb + (p.zr != nullptr ? zb : 0u));
      if (ntok > 0) mbar_expect_tx(bar_act, total);
      for (int t = 0; t < ntok; ++t) {
        if constexpr (PAIR)
          bulk_g2s(smem_u32(sA + t * p.a_stride), p.qsp + (size_t)(p.m0 + t) * (p.kpad / 64) * 80, alen, bar_act);
        else
          bulk_g2s(smem_u32(sA + t * p.a_stride), p.qs + (size_t)(p.m0 + t) * p.kpad, alen, bar_act);
        bulk_g2s(smem_u32(sDS + (size_t)t * p.nb32tot), p.ds + (size_t)(p.m0 + t) * p.nb32tot, dsb, bar_act);
        if (p.zr != nullptr)
          bulk_g2s(smem_u32(sZ + (size_t)t * p.nb32tot * p.zpb), p.zr + (size_t)(p.m0 + t) * p.nb32tot * p.zpb, zb, bar_act);
      }
      bool ok = true;
      for (; q < nstages; ++q) {
        if (q >= S) ok = mbar_wait(bar_empty + 8 * (q % S), (uint32_t)((q / S - 1) & 1), s_abort);
        if (!ok) break;
        issue_stage(q);
      }
      const int first = q > S ? q - S : 0;
      for (int qq = first; qq < q; ++qq) mbar_wait(bar_full + 8 * (qq % S), (uint32_t)((qq / S) & 1), s_abort);
      if (!ok) atomicExch(p.status, 1);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  if (p.x != nullptr) {
    pdl_wait();                                   // x may come from the kernel before this one
    // no quantizer launch clears the status word of this scratch: do it here, after the previous kernel (which may
    // still report into it) has finished
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.m0 == 0) *p.status = 0;
    quantize_rows_smem<PAIR>(p, sA, sDS, sZ, warp, lane, p.mcount < MT ? p.mcount : MT);
    asm volatile("bar.sync 2, %0;" ::"n"(ROW_WARPS * 32) : "memory");   // all sixteen consumer warps, nobody has left yet
  } else if (!mbar_wait(bar_act, 0, s_abort)) {
    if (lane == 0) atomicExch(p.status, 2);
    return;
  }
  OutT* y = reinterpret_cast<OutT*>(p.y);
  constexpr int NG = 32 / F::GROUP;
  const int zmode = p.zmode;
  if constexpr (PAIR) {
    static_assert(!PAIR || QT == KQ_TYPE_Q4_K || QT == KQ_TYPE_Q6_K, "pair mode is written for Q4_K and Q6_K");
    const int npairs = (r1 - r0 + 1) / 2;
    const int ri = lane >> 4, sbo = (lane >> 2) & 3, il = lane & 3;
    const int nsb8 = p.nsb >> 3;
    for (int j = warp; j < npairs; j += ROW_WARPS) {
      const int i = 2 * j;
      const int q = i / R, slot = q % S;
      if (*s_issued <= q) {
        const long long t0 = clock64();
        while (*s_issued <= q) {
          if (*s_abort || clock64() - t0 > WAIT_LIMIT) { *s_abort = 1; if (lane == 0) atomicExch(p.status, 4); return; }
        }
      }
      if (!mbar_wait(bar_full + 8 * slot, (uint32_t)((q / S) & 1), s_abort)) { if (lane == 0) atomicExch(p.status, 3); return; }
      const int row = r0 + i + ri;
      const bool valid_row = row < r1;
      const uint32_t off = (uint32_t)((uintptr_t)(p.W + (size_t)(r0 + q * R) * p.rowbytes) & 15);
      const uint8_t* prow = ring + (size_t)slot * p.stage_bytes + off + (size_t)(i - q * R + ri) * p.rowbytes;
      float acc[MT];
#pragma unroll
      for (int t = 0; t < MT; ++t) acc[t] = 0.f;
      if (valid_row) {
        if constexpr (QT == KQ_TYPE_Q4_K) {
        for (int s = sbo; s < nsb8; s += 4) {
          const uint8_t* bp = prow + (size_t)s * 144;
          const uint4 hdr = *reinterpret_cast<const uint4*>(bp);
          const uint32_t scw = il < 2 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u));
          const uint32_t mnw = il < 2 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u));
          const int sh = 16 * (il & 1);
          const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
          const float dl = dm.x * (float)((scw >> sh) & 0xFFu);
          const float dh = dm.x * (float)((scw >> (sh + 8)) & 0xFFu) * 0.0625f;   // high nibbles are used as 16*q
          const float ml = dm.y * (float)((mnw >> sh) & 0xFFu);
          const float mh = dm.y * (float)((mnw >> (sh + 8)) & 0xFFu);
          const uint4 w0 = *reinterpret_cast<const uint4*>(bp + 16 + 32 * il);
          const uint4 w1 = *reinterpret_cast<const uint4*>(bp + 32 + 32 * il);
          const uint32_t wq[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) { lo[k] = wq[k] & 0x0F0F0F0Fu; hi[k] = wq[k] & 0xF0F0F0F0u; }
          const int b = s * 8 + 2 * il;
#pragma unroll
          for (int t = 0; t < MT; ++t) {
            const uint4* ap = reinterpret_cast<const uint4*>(sA + (size_t)t * p.a_stride + (size_t)(s * 4 + il) * 80);
            const uint4 a0 = ap[0], a1 = ap[1], a2 = ap[2], a3 = ap[3];
            const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint32_t ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
            int Il = 0, Ih = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) { Il = __dp4a((int)lo[k], (int)al[k], Il); Ih = dp4a_us(hi[k], ah[k], Ih); }
            const uint2 dsw = *reinterpret_cast<const uint2*>(sDS + (size_t)t * p.nb32tot + b);
            const float2 dsl = __half22float2(*reinterpret_cast<const __half2*>(&dsw.x));
            const float2 dsh = __half22float2(*reinterpret_cast<const __half2*>(&dsw.y));
            float zl = dsl.y, zh = dsh.y;
            if (zmode != 1) {
              const float2 z = *reinterpret_cast<const float2*>(sZ + (size_t)t * p.nb32tot + b);
              zl = z.x; zh = z.y;
            }
            acc[t] += dl * (dsl.x * (float)Il) + dh * (dsh.x * (float)Ih) - (ml * zl + mh * zh);
          }
        }
        } else {
        // Q6_K: lane = (row of the pair, super-block offset, part = (ip, ilh)); a part is 64 weights: for
        // q4 = 0..3 the 16 weights 128ip + 32q4 + 16ilh .. of the super-block, i.e. 16 bytes of ql's first half
        // (low nibbles -> q4=0, high -> q4=2), 16 bytes of its second half (q4=1, 3) and 16 bytes of qh.
        // The 6-bit codes stay unsigned (u8 x s8 dp4a); the -32 offset is applied as -32 * d8 * sum(codes of the
        // activation group), read from the token-major z16r table.
        const int ip = il >> 1, ilh = il & 1;
        for (int s = sbo; s < nsb8; s += 4) {
          const uint8_t* bp = prow + (size_t)s * 210;
          const uint8_t* pa = bp + 64 * ip + 16 * ilh;
          // the three 16-byte runs sit 32 and 128-32ip-... bytes apart: same alignment phase; fetch aligned words
          const uintptr_t a_al = (uintptr_t)pa & ~(uintptr_t)3;
          const int shb = (int)((uintptr_t)pa & 3) * 8;         // 0 or 16 bits
          const uint32_t* wa = reinterpret_cast<const uint32_t*>(a_al);
          const uint32_t* wb = reinterpret_cast<const uint32_t*>(a_al + 32);
          const uint32_t* wh = reinterpret_cast<const uint32_t*>(a_al + (128 + 32 * ip + 16 * ilh) - (64 * ip + 16 * ilh));
          uint32_t A[4], B[4], H[4];
          {
            uint32_t ra[5], rb[5], rh[5];
#pragma unroll
            for (int w = 0; w < 5; ++w) { ra[w] = wa[w]; rb[w] = wb[w]; rh[w] = wh[w]; }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              A[w] = __funnelshift_r(ra[w], ra[w + 1], shb);
              B[w] = __funnelshift_r(rb[w], rb[w + 1], shb);
              H[w] = __funnelshift_r(rh[w], rh[w + 1], shb);
            }
          }
          uint32_t q[4][4];   // [q4][word]
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            q[0][w] = (A[w] & 0x0F0F0F0Fu) | ((H[w] << 4) & 0x30303030u);
            q[1][w] = (B[w] & 0x0F0F0F0Fu) | ((H[w] << 2) & 0x30303030u);
            q[2][w] = ((A[w] >> 4) & 0x0F0F0F0Fu) | (H[w] & 0x30303030u);
            q[3][w] = ((B[w] >> 4) & 0x0F0F0F0Fu) | ((H[w] >> 2) & 0x30303030u);
          }
          const float d = ld_h(bp + 208);
          float wsc[4];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) wsc[q4] = d * (float)(int8_t)bp[192 + 8 * ip + 2 * q4 + ilh];
          const int b = s * 8 + 4 * ip;      // first of the part's four 32-blocks
#pragma unroll
          for (int t = 0; t < MT; ++t) {
            const uint8_t* ap = sA + (size_t)t * p.a_stride + (size_t)(s * 4 + 2 * ip) * 80 + 16 * ilh;
            const uint4 a0 = *reinterpret_cast<const uint4*>(ap);            // q4 = 0
            const uint4 a1 = *reinterpret_cast<const uint4*>(ap + 32);       // q4 = 1
            const uint4 a2 = *reinterpret_cast<const uint4*>(ap + 80);       // q4 = 2
            const uint4 a3 = *reinterpret_cast<const uint4*>(ap + 112);      // q4 = 3
            const uint32_t aw[4][4] = {{a0.x, a0.y, a0.z, a0.w}, {a1.x, a1.y, a1.z, a1.w}, {a2.x, a2.y, a2.z, a2.w}, {a3.x, a3.y, a3.z, a3.w}};
            const uint4 dsw = *reinterpret_cast<const uint4*>(sDS + (size_t)t * p.nb32tot + b);
            const uint32_t dsr[4] = {dsw.x, dsw.y, dsw.z, dsw.w};
            const float* zp = sZ + ((size_t)t * p.nb32tot + b) * 2 + ilh;
            float c = 0.f;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              int I = 0;
#pragma unroll
              for (int w = 0; w < 4; ++w) I = dp4a_us(q[q4][w], aw[q4][w], I);
              const float d8 = __low2float(*reinterpret_cast<const __half2*>(&dsr[q4]));
              c += wsc[q4] * (d8 * (float)I - 32.0f * zp[2 * q4]);
            }
            acc[t] += c;
          }
        }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
#pragma unroll
      for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int mask = 8; mask > 0; mask >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], mask);
      }
      float mine = 0.f;
#pragma unroll
      for (int t = 0; t < MT; ++t) if ((lane & 15) == t) mine = acc[t];
      if (valid_row && (lane & 15) < MT && (lane & 15) < p.mcount)
        y[(size_t)(p.m0 + (lane & 15)) * p.stride_y + row] = from_f32<OutT>(mine);
    }
    return;
  } else {
  for (int i = warp; r0 + i < r1; i += ROW_WARPS) {
    const int row = r0 + i;
    const int q = i / R, slot = q % S;
    if (*s_issued <= q) {   // the slot's barrier may still show an older generation until stage q is issued
      const long long t0 = clock64();
      while (*s_issued <= q) {
        if (*s_abort || clock64() - t0 > WAIT_LIMIT) { *s_abort = 1; if (lane == 0) atomicExch(p.status, 4); return; }
      }
    }
    if (!mbar_wait(bar_full + 8 * slot, (uint32_t)((q / S) & 1), s_abort)) { if (lane == 0) atomicExch(p.status, 3); return; }
    const uint32_t off = (uint32_t)((uintptr_t)(p.W + (size_t)(r0 + q * R) * p.rowbytes) & 15);
    const uint8_t* prow = ring + (size_t)slot * p.stage_bytes + off + (size_t)(i - q * R) * p.rowbytes;
    float acc[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[t] = 0.f;
    const int swz = (lane >> 2) & 1;
    for (int sb = lane; sb < p.nsb; sb += 32) {
      SubBlock s;
      decode_subblock<QT>(prow, sb, s_grid, s);
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        const uint8_t* ap = sA + (size_t)t * p.a_stride + sb * 32;
        const uint4 ua = *reinterpret_cast<const uint4*>(ap + 16 * swz);
        const uint4 ub = *reinterpret_cast<const uint4*>(ap + 16 * (swz ^ 1));
        const uint4 u0 = swz ? ub : ua, u1 = swz ? ua : ub;
        const uint32_t u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        const float2 dsf = __half22float2(sDS[(size_t)t * p.nb32tot + sb]);
        const float d8 = dsf.x;
        int I[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int hh = (NG == 2) ? (j >> 2) : 0;
          I[hh] = __dp4a((int)s.v[j], (int)u[j], I[hh]);
        }
        float c;
        if constexpr (HalfProd<QT>::value) {
          // d * d8 and m * s8 rounded to fp16 first, as the reference's __hmul2 does (wb holds -m)
          c = __half2float(__float2half_rn(s.wa[0] * d8)) * (float)I[0] - __half2float(__float2half_rn(s.wb[0] * dsf.y));
        } else if constexpr (NG == 1) {
          c = s.wa[0] * (d8 * (float)I[0]);
          if constexpr (F::HAS_MIN) c -= s.wb[0] * (zmode == 1 ? dsf.y : sZ[(size_t)t * p.nb32tot + sb]);
        } else {
          c = d8 * (s.wa[0] * (float)I[0] + s.wa[1] * (float)I[1]);
          if constexpr (F::HAS_MIN) {
            const float2 z = *reinterpret_cast<const float2*>(sZ + ((size_t)t * p.nb32tot + sb) * 2);
            c -= s.wb[0] * z.x + s.wb[1] * z.y;
          }
        }
        acc[t] += c;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * slot);   // this row's bytes are no longer needed
#pragma unroll
    for (int t = 0; t < MT; ++t) {
#pragma unroll
      for (int mask = 16; mask > 0; mask >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], mask);
    }
    float mine = 0.f;
#pragma unroll
    for (int t = 0; t < MT; ++t) if (lane == t) mine = acc[t];
    if (lane < MT && lane < p.mcount) y[(size_t)(p.m0 + lane) * p.stride_y + row] = from_f32<OutT>(mine);
  }
  }
}

// ---------------------------------------------------------------------------------------------- host
// ---------------------------------------------------------------------------------------------- host
struct RowConfig {
  int rows_per_stage, stages, stage_bytes, a_stride, a_bytes, d_bytes, z_bytes, smem, grid;
};

int z_per_block(int type) {
  if (type == KQ_TYPE_Q2_K) return 2;
  return (type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q4_0 || type == KQ_TYPE_Q5_K || type == KQ_TYPE_Q5_0) ? 1 : 0;
}

constexpr int SMEM_LIMIT = 227 * 1024;

// row-streaming kernel: whole rows per stage, the full K of `mt` tokens resident in shared memory
bool make_row_config(int type, int64_t n, int64_t k, int mt, bool pair, RowConfig& c) {
  int blk, bytes;
  if (!type_geometry(type, &blk, &bytes)) return false;
  const int64_t rowbytes = k / blk * bytes;
  const int zpb = z_per_block(type);
  // Stage size.  The producer lane's loop is the request rate of an SM, so the Q4_K row-pair kernel, whose 16 KB target
  // gave 11.5 KB stages (an even number of 2880-byte rows), runs on 24 KB stages: 15.3 -> 13.1 us on 17408x5120 at one
  // token, 28.2 -> 21.3 us on 34816x5120.  The one-row-per-warp kernels were not faster with larger stages (Q8_0
  // 5120x5120 at two tokens: 10.3 -> 12.2 us), they keep 16 KB.
  const int64_t stage_target = (pair && type == KQ_TYPE_Q4_K) ? (int64_t)options().row_stage_kb * 1024 : 16384;
  int R = (int)(stage_target / rowbytes);
  if (R < 1) R = 1;
  if (R > 32) R = 32;
  if (pair) R = R < 2 ? 2 : (R & ~1);   // a warp's two rows never straddle stages
  c.rows_per_stage = R;
  c.stage_bytes = (int)((R * rowbytes + 32 + 127) / 128 * 128);
  const int64_t kpad = (k + 511) / 512 * 512;
  const bool zr = type == KQ_TYPE_Q2_K || type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q5_K || type == KQ_TYPE_Q5_0 ||
                  (pair && type == KQ_TYPE_Q6_K);
  c.a_stride = pair ? (int)(k / 64) * 80 + 16 : (int)k + 32;
  c.a_bytes = (mt * c.a_stride + 127) / 128 * 128;
  c.d_bytes = (int)((mt * (kpad / 32) * 4 + 127) / 128 * 128);
  c.z_bytes = zr ? (int)((mt * (kpad / 32) * 4 * ((type == KQ_TYPE_Q2_K || type == KQ_TYPE_Q6_K) ? 2 : 1) + 127) / 128 * 128) : 0;
  (void)zpb;
  const int fixed = SMEM_HEADER + (type == KQ_TYPE_IQ3_S ? 2048 : 0) + c.a_bytes + c.d_bytes + c.z_bytes;
  if (fixed + 3 * (int64_t)c.stage_bytes > SMEM_LIMIT) return false;
  int stages = (SMEM_LIMIT - fixed) / c.stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  c.stages = stages;
  c.smem = fixed + stages * c.stage_bytes;
  const int sms = sm_count();
  c.grid = n < sms ? (int)n : sms;
  return true;
}

template <int QT, int MT, bool PAIR, typename OutT>
int launch_rows(const RowParams& p, const RowConfig& c, cudaStream_t st) {
  auto kern = gemv_rows_kernel<QT, MT, PAIR, OutT>;
  static DeviceOnce attr_set;   // the attribute belongs to the (function, device) pair
  if (attr_set.first_time()) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    attr_set.done();
  }
  KQ_CUDA_TRY(launch_pdl(kern, dim3(c.grid), dim3(ROW_THREADS), (size_t)c.smem, st, options().pdl != 0, p));
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT, typename OutT>
int launch_rows_mt(const RowParams& p, const RowConfig& c, int mt, cudaStream_t st) {
  if constexpr (QT == KQ_TYPE_Q4_K || QT == KQ_TYPE_Q6_K) {
    if (p.qsp != nullptr) {
      switch (mt) {
        case 1: return launch_rows<QT, 1, true, OutT>(p, c, st);
        case 2: return launch_rows<QT, 2, true, OutT>(p, c, st);
        case 4: return launch_rows<QT, 4, true, OutT>(p, c, st);
        default: return launch_rows<QT, 8, true, OutT>(p, c, st);
      }
    }
  }
  switch (mt) {
    case 1: return launch_rows<QT, 1, false, OutT>(p, c, st);
    case 2: return launch_rows<QT, 2, false, OutT>(p, c, st);
    case 4: return launch_rows<QT, 4, false, OutT>(p, c, st);
    default: return launch_rows<QT, 8, false, OutT>(p, c, st);
  }
}

template <int QT>
int launch_typed(const RowParams& p, const RowConfig& c, int mt, int y_dtype, cudaStream_t st) {
  switch (y_dtype) {
    case KQ_F32: return launch_rows_mt<QT, float>(p, c, mt, st);
    case KQ_F16: return launch_rows_mt<QT, __half>(p, c, mt, st);
    case KQ_BF16: return launch_rows_mt<QT, __nv_bfloat16>(p, c, mt, st);
  }
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace

// The streaming kernels fetch weights in 16-byte units, so they need a 16-byte aligned weight pointer; anything
// else goes to the general dp4a kernel.
bool gemv_mma_supported(const void* W, int type, int64_t n, int64_t k) {
  if ((uintptr_t)W % 16) return false;
  RowConfig c;
  return make_row_config(type, n, k, 1, false, c);
}

// Smallest token count that goes to the shared-stage mma kernel in auto mode.  Q4_0's 18-byte blocks decode slowly
// there (row-streaming kernel up to 8 tokens).  Q6_K's row-streaming consumer tops out near 3 TB/s, the mma kernel
// near 4.2 TB/s, so whenever it needs no K split (K up to about 8K) the mma kernel takes 1-2 tokens as well: 27.2 ->
// 21.0 us on 17408x5120, 352 -> 246 us on a 248320x5120 LM head; with a K split (5120x17408) the row kernel stays ahead.
static int tile_min_tokens(int type, int64_t n, int64_t k) {
  if (!type_is_core(type)) return 1 << 30;   // the other formats never leave the row-streaming kernel
  if (type == KQ_TYPE_Q4_0) return 9;
  if (type == KQ_TYPE_Q6_K && gemv_tile_splits(type, n, k, 8) == 1) return 1;
  if (type == KQ_TYPE_IQ3_S) return 2;   // its generic row decoder pays per token: 29.4 -> 27.0 us at 2 tokens
  return options().tc_min_m;
}

// True when every token of an m-token call goes to the row-streaming kernel (which can quantize raw activations itself).
bool gemv_rows_only(int type, int64_t n, int64_t k, int64_t m) {
  const int impl = options().gemv_impl;
  if (impl == 3 || impl == 4) return true;
  if (impl != 0) return false;
  return m < tile_min_tokens(type, n, k);
}

// impl: 0 = choose by m, 3 = row-streaming dp4a, 4 = the same without the specialised consumers, 6 = shared-stage mma
// fuse_x != nullptr (only with gemv_rows_only): the activations have NOT been quantized into P; the kernel reads them raw
int launch_gemv_mma(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m, void* y, int y_dtype,
                    int64_t stride_y, bool mmq, cudaStream_t st, const void* fuse_x, int x_dtype, int64_t stride_x) {
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  const int impl = options().gemv_impl;
  if (impl == 2 || impl == 5) { set_error("gemv_impl %d names a kernel that is no longer part of the library", impl); return KQ_EUNSUPPORTED; }
  const int zpb = z_per_block(type) ? z_per_block(type) : 1;
  int64_t m0 = 0;
  while (m0 < m) {
    const int64_t left = m - m0;
    const bool tile_start = (m0 % 16) == 0;
    int rc, mcount;
    const int tile_min = tile_min_tokens(type, n, k);
    // 3..16 tokens: the register-resident mma kernel where it covers the type and shape
    // (today it wins for up to 8 tokens; 9..16 tokens only on request: kres = 2 or gemv_impl = 7)
    const int pass = (int)(left < 16 ? left : 16);
    // the tensor-memory kernel (tcgen05 integer MMAs): on request for now (gemv_impl = 8, or option umma = 1 in auto mode)
    if (tile_start && (impl == 8 || (impl == 0 && options().umma && left >= options().umma_min_m)) && gemv_umma_supported(W, type, n, k)) {
      mcount = pass;
      rc = launch_gemv_umma(W, type, n, k, P, m0, mcount, y, y_dtype, stride_y, mmq, st);
      if (rc) return rc;
      m0 += mcount;
      continue;
    }
    if (impl == 8) { set_error("tensor-memory GEMV: type/shape not covered"); return KQ_EUNSUPPORTED; }
    if (tile_start && (impl == 7 || (impl == 0 && left >= tile_min && (options().kres == 2 || (options().kres == 1 && pass <= 8)))) &&
        gemv_kres_supported(W, type, n, k, pass)) {
      mcount = (int)(left < 16 ? left : 16);
      rc = launch_gemv_kres(W, type, n, k, P, m0, mcount, y, y_dtype, stride_y, mmq, st);
      if (rc) return rc;
      m0 += mcount;
      continue;
    }
    if (impl == 7) { set_error("register-resident GEMV: type/shape not covered"); return KQ_EUNSUPPORTED; }
    // otherwise the shared-stage mma kernel (all warps of a CTA on every stage of 8 rows)
    if (tile_start && (impl == 6 || (impl == 0 && left >= tile_min)) &&
        gemv_tile_supported(W, type, n, k, (int)(left < 16 ? left : 16))) {
      mcount = (int)(left < 16 ? left : 16);
      rc = launch_gemv_tile(W, type, n, k, P, m0, mcount, y, y_dtype, stride_y, mmq, st);
      if (rc) return rc;
      m0 += mcount;
      continue;
    }
    if (impl == 6) { set_error("tile GEMV: type/shape not covered"); return KQ_EUNSUPPORTED; }
    const int room = 16 - (int)(m0 % 16);          // a pass never crosses a 16-token tile of the scale tables
    const int cap = (int)(left < room ? left : room);
    int mt = cap >= 8 ? 8 : (cap >= 4 ? 4 : (cap >= 2 ? 2 : 1));
    RowConfig rcg;
    // specialised consumers: Q4_K always; Q6_K only for 1-2 tokens (its per-token cost is higher than the general one's)
    const bool pair = impl != 4 && (k % 256) == 0 && (type == KQ_TYPE_Q4_K || (type == KQ_TYPE_Q6_K && mt <= 2));
    while (mt > 1 && !make_row_config(type, n, k, mt, pair, rcg)) mt >>= 1;   // fewer tokens per pass if K is long
    if (!make_row_config(type, n, k, mt, pair, rcg)) { set_error("row-streaming GEMV: no configuration for this shape"); return KQ_EUNSUPPORTED; }
    mcount = mt;
    RowParams p;
    p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.n = (int)n; p.nsb = (int)(k / 32);
    p.rows_per_stage = rcg.rows_per_stage; p.stages = rcg.stages; p.stage_bytes = rcg.stage_bytes;
    p.a_stride = rcg.a_stride; p.a_bytes = rcg.a_bytes; p.d_bytes = rcg.d_bytes; p.z_bytes = rcg.z_bytes;
    p.qs = P.qs; p.qsp = pair ? P.qsp : nullptr; p.ds = P.ds; p.zpb = zpb; p.kpad = (int)P.kpad; p.nb32tot = (int)(P.kpad / 32); p.klen = (int)k;
    p.zr = nullptr; p.zmode = 0;
    // min term: the fp16 raw block sum (mode 1) or d8 * (sum of the codes) from the token-major table (mode 2)
    if (type == KQ_TYPE_Q4_0 || type == KQ_TYPE_Q4_1 || type == KQ_TYPE_Q5_1 || ((type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q5_K) && mmq) ||
        (type == KQ_TYPE_Q5_0 && !mmq)) p.zmode = 1;
    else if (type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q5_K || type == KQ_TYPE_Q5_0) { p.zmode = 2; p.zr = P.z32r; }
    else if (type == KQ_TYPE_Q2_K) { p.zmode = 3; p.zr = P.z16r; }
    else if (type == KQ_TYPE_Q6_K && pair) { p.zmode = 3; p.zr = P.z16r; p.zpb = 2; }   // -32 offset via group sums
    p.prefetch = options().pdl < rcg.stages ? options().pdl : rcg.stages;
    p.m0 = (int)m0; p.mcount = mcount; p.y = y; p.stride_y = stride_y; p.status = P.status;
    p.x = fuse_x; p.x_dtype = x_dtype; p.stride_x = stride_x;
    switch (type) {
      case KQ_TYPE_Q4_0: rc = launch_typed<KQ_TYPE_Q4_0>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q8_0: rc = launch_typed<KQ_TYPE_Q8_0>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q2_K: rc = launch_typed<KQ_TYPE_Q2_K>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q4_K: rc = launch_typed<KQ_TYPE_Q4_K>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q6_K: rc = launch_typed<KQ_TYPE_Q6_K>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_IQ3_S: rc = launch_typed<KQ_TYPE_IQ3_S>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q4_1: rc = launch_typed<KQ_TYPE_Q4_1>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q5_0: rc = launch_typed<KQ_TYPE_Q5_0>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q5_1: rc = launch_typed<KQ_TYPE_Q5_1>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q3_K: rc = launch_typed<KQ_TYPE_Q3_K>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_Q5_K: rc = launch_typed<KQ_TYPE_Q5_K>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_IQ4_NL: rc = launch_typed<KQ_TYPE_IQ4_NL>(p, rcg, mt, y_dtype, st); break;
      case KQ_TYPE_IQ4_XS: rc = launch_typed<KQ_TYPE_IQ4_XS>(p, rcg, mt, y_dtype, st); break;
      default: set_error("row-streaming GEMV: type %d not covered", type); return KQ_EUNSUPPORTED;
    }
    if (rc) return rc;
    m0 += mcount;
  }
  return KQ_OK;
}

}  // namespace kq
