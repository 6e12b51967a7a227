// Decode GEMV: the dispatch over the streaming kernels (launch_gemv_mma, bottom of the file) and two of them:
//   gemv_rows_kernel    1-2 tokens (and every count for shapes the shared-stage kernel does not take): whole rows per
//                       stage, dp4a consumers, optional in-kernel q8_1 quantization; described above its definition
//   gemv_stream_kernel  the first int8 mma.sync kernel (a warp owns a 16-row tile), kept behind gemv_impl=2 for
//                       comparison; described here.  The default for 3..80 tokens is kq_gemv_tile.cu.
//
//   grid      one CTA per SM (148), split into `ks` groups; group s works on the K range of split s
//   CTA       8 consumer warps + 1 producer warp
//   producer  bulk-copies (cp.async.bulk, completion on an mbarrier) the CTA's slice of the quantized
//             activations once, then feeds a ring of stages; one stage = 16 consecutive weight rows x `cb`
//             wire blocks, fetched as 16 row segments (each start rounded down / end rounded up to 16 bytes)
//   consumer  a warp owns a whole 16-row tile: it consumes the tile's stages in order, keeps the 16 x M
//             partial sums in registers (mma C-fragment layout) and writes the tile's outputs itself, so
//             consumer warps never synchronise with each other
//   mma       weights are the A operand (16 rows x 32 or 16 k), tokens the B operand (8 per n-tile).  The
//             position of a weight inside a 32-block is permuted freely as long as the activation fragment is
//             read with the same permutation, so a lane's nibbles unpack with two logic ops per register.
//   split-K   when ks > 1 every warp writes fp32 partials for its (tile, split); the last split to arrive
//             at the tile's counter adds them in split order (deterministic) and stores the outputs.
//
// The integer dots are exact; the fp32 combine follows the reference's vec_dot functions
// (vllm_gguf_plugin/csrc/gguf/vecdotq.cuh:328-379 Q4_K, 447-491 Q6_K).
//
// A consumer may be several ring generations ahead of the producer (its next tile can map to a slot whose
// previous fills belong to other warps), and an mbarrier parity test cannot tell generation f from f-2.  So
// the producer publishes the number of stages it has issued and a consumer looks at the slot's barrier
// only once its own stage has been issued; from then on the barrier is at most one phase behind.
//
// Every wait is bounded: after ~2^27 clocks the waiter raises a CTA-wide abort flag and a
// status word in global memory, every warp leaves its loop, and the producer waits (again bounded) for
// the copies it has in flight before the CTA exits.
#include "kq_common.cuh"

namespace kq {

namespace {

constexpr int TILE_ROWS = 16;
// consumer warps: tensor-core mode 8 (a warp owns a tile); dp4a mode 16 (a warp owns one row of every tile)
__host__ __device__ constexpr int consumer_warps(int mode) { return mode == 0 ? 8 : 16; }
// producer warps of the tensor-core kernel: the copy engine takes requests faster from several warps (4 lanes of
// 4 warps: ~20 ns per request and SM; 16 lanes of one warp: ~40 ns), and a row segment is only 1-2 KB
constexpr int NPROD = 4;
__host__ __device__ constexpr int cta_threads(int mode) { return (consumer_warps(mode) + (mode == 0 ? NPROD : 1)) * 32; }
constexpr uint32_t MAGIC_I = 0x4B400000u;  // bits of 12582912.0f: adding an int |v| < 2^22 gives the float 12582912+v
constexpr float MAGIC_F = 12582912.0f;
constexpr long long WAIT_LIMIT = 1ll << 27;   // ~70 ms at 1.9 GHz; a healthy wait lasts microseconds
constexpr int SMEM_HEADER = 1024;
constexpr int MAX_STAGES = 32;

__constant__ uint16_t c_iq3s_codes_s[512] = {
#include "kq_iq3s_codes.inc"
};

struct MmaParams {
  const uint8_t* W;
  int64_t rowbytes;
  int n, nblk, ks, ntiles, cb, stages, slot_stride, stage_bytes;
  int a_stride, a_bytes, d_bytes, z_bytes;
  const int8_t* qs;
  const float* dT;
  const float* zT;   // min-term table of this type/flavour (nullptr if the type has none)
  int zpb;           // z entries per 32-block (1 or 2)
  int kpad, nb32tot;
  int m0, mcount;
  int prefetch;      // ring stages each producer issues before it waits for the previous kernel
  void* y;
  int64_t stride_y;
  float* part;
  int* cnt;
  int* status;
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

__device__ __forceinline__ void mma_s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// 32 bits from a 2-byte aligned shared-memory address (two aligned words + byte permute)
__device__ __forceinline__ uint32_t lds32_a2(const uint8_t* p) {
  const uintptr_t a = (uintptr_t)p;
  const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~(uintptr_t)3);
  const uint32_t lo = q[0], hi = q[1];
  return __byte_perm(lo, hi, (a & 2) ? 0x5432 : 0x3210);
}
__device__ __forceinline__ int sext_byte(uint32_t w, int i) { return (int)(int8_t)(w >> (8 * i)); }

// exact int -> float for |v| < 2^22 without the conversion pipe
__device__ __forceinline__ float magic_float(int v) { return __int_as_float(v + (int)MAGIC_I) - MAGIC_F; }

struct ActView {   // the CTA's slice of the quantized activations in shared memory
  const uint8_t* sA;  // [8*NT tokens][a_stride] codes
  int a_stride;
  const float* sD;    // [32-block][16 tokens]
  const float* sZ;    // [z entry][16 tokens]
};

// ---------------------------------------------------------------------------------------------- Q4_K
// pg/ph: first byte of this chunk's blocks for rows g and g+8; b0: index of the chunk's first 32-block inside
// the CTA's K range.  Lane (g,t) covers codes 8t..8t+7 of every 32-weight sub-block (one 64-bit load yields
// the low-nibble sub-block 2*il and the high-nibble sub-block 2*il+1).
template <int NT>
__device__ __forceinline__ void chunk_q4k(const uint8_t* pg, const uint8_t* ph, int nblocks, int b0, const ActView& A,
                                          int g, int t, float (&acc)[NT][4]) {
  for (int sbi = 0; sbi < nblocks; ++sbi) {
    const uint8_t* bg = pg + sbi * 144;
    const uint8_t* bh = ph + sbi * 144;
    const uint32_t* hg = reinterpret_cast<const uint32_t*>(bg);
    const uint32_t* hh = reinterpret_cast<const uint32_t*>(bh);
    const uint32_t g0 = hg[1], g1 = hg[2], g2 = hg[3];
    const uint32_t h0 = hh[1], h1 = hh[2], h2 = hh[3];
    // 6-bit scales / mins as bytes: lo = sub-blocks 0-3, hi = 4-7 (reference: dequantize.cuh:156-163)
    const uint32_t scg[2] = {g0 & 0x3F3F3F3Fu, (g2 & 0x0F0F0F0Fu) | ((g0 >> 2) & 0x30303030u)};
    const uint32_t mng[2] = {g1 & 0x3F3F3F3Fu, ((g2 >> 4) & 0x0F0F0F0Fu) | ((g1 >> 2) & 0x30303030u)};
    const uint32_t sch[2] = {h0 & 0x3F3F3F3Fu, (h2 & 0x0F0F0F0Fu) | ((h0 >> 2) & 0x30303030u)};
    const uint32_t mnh[2] = {h1 & 0x3F3F3F3Fu, ((h2 >> 4) & 0x0F0F0F0Fu) | ((h1 >> 2) & 0x30303030u)};
    float u[NT][4], um[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) { u[nt][i] = 0.f; um[nt][i] = 0.f; }
#pragma unroll
    for (int il = 0; il < 4; ++il) {
      const uint2 wg = *reinterpret_cast<const uint2*>(bg + 16 + 32 * il + 8 * t);
      const uint2 wh = *reinterpret_cast<const uint2*>(bh + 16 + 32 * il + 8 * t);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * il + e;
        const uint32_t a0 = (wg.x >> (4 * e)) & 0x0F0F0F0Fu, a2 = (wg.y >> (4 * e)) & 0x0F0F0F0Fu;
        const uint32_t a1 = (wh.x >> (4 * e)) & 0x0F0F0F0Fu, a3 = (wh.y >> (4 * e)) & 0x0F0F0F0Fu;
        const int sg = (int)((scg[j >> 2] >> (8 * (j & 3))) & 0xFFu);
        const int sh = (int)((sch[j >> 2] >> (8 * (j & 3))) & 0xFFu);
        const float mg = (float)((mng[j >> 2] >> (8 * (j & 3))) & 0xFFu);
        const float mh = (float)((mnh[j >> 2] >> (8 * (j & 3))) & 0xFFu);
        const int b = b0 + sbi * 8 + j;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint2 bb = *reinterpret_cast<const uint2*>(A.sA + (8 * nt + g) * A.a_stride + b * 32 + 8 * t);
          int D[4];
          mma_s8_k32(D, a0, a1, a2, a3, bb.x, bb.y);
          const float2 d8 = *reinterpret_cast<const float2*>(A.sD + b * 16 + 8 * nt + 2 * t);
          const float2 z = *reinterpret_cast<const float2*>(A.sZ + b * 16 + 8 * nt + 2 * t);
          u[nt][0] = fmaf(magic_float(D[0] * sg), d8.x, u[nt][0]);   // |dot * sc| <= 60960 * 63 < 2^22
          u[nt][1] = fmaf(magic_float(D[1] * sg), d8.y, u[nt][1]);
          u[nt][2] = fmaf(magic_float(D[2] * sh), d8.x, u[nt][2]);
          u[nt][3] = fmaf(magic_float(D[3] * sh), d8.y, u[nt][3]);
          um[nt][0] = fmaf(mg, z.x, um[nt][0]);
          um[nt][1] = fmaf(mg, z.y, um[nt][1]);
          um[nt][2] = fmaf(mh, z.x, um[nt][2]);
          um[nt][3] = fmaf(mh, z.y, um[nt][3]);
        }
      }
    }
    const float2 dmg = __half22float2(*reinterpret_cast<const __half2*>(&hg[0]));
    const float2 dmh = __half22float2(*reinterpret_cast<const __half2*>(&hh[0]));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc[nt][0] += dmg.x * u[nt][0] - dmg.y * um[nt][0];
      acc[nt][1] += dmg.x * u[nt][1] - dmg.y * um[nt][1];
      acc[nt][2] += dmh.x * u[nt][2] - dmh.y * um[nt][2];
      acc[nt][3] += dmh.x * u[nt][3] - dmh.y * um[nt][3];
    }
  }
}

// ---------------------------------------------------------------------------------------------- Q6_K
// 16-weight scale groups -> m16n8k16.  Group (ip, q4, s) holds weights 128ip+32q4+16s+4t.. of the super-block:
// low nibbles from ql[64ip + 32(q4&1) + 16s + 4t], 2 high bits from qh[32ip + 16s + 4t] >> 2q4.  The two
// groups s=0,1 of one 32-block share the activation scale, so their scaled dots are added as integers first
// (as the reference's MMQ kernel does, vecdotq.cuh:467-491); |sum| < 2^24, so the conversion is exact.
__device__ __forceinline__ uint32_t unpack6(uint32_t qlw, uint32_t qhw, int q4) {
  const uint32_t lo = (qlw >> (4 * (q4 >> 1))) & 0x0F0F0F0Fu;
  const uint32_t hi = ((qhw >> (2 * q4)) & 0x03030303u) << 4;
  return sub32_bytes(lo | hi);
}

template <int NT>
__device__ __forceinline__ void chunk_q6k(const uint8_t* pg, const uint8_t* ph, int nblocks, int b0, const ActView& A,
                                          int g, int t, float (&acc)[NT][4]) {
  for (int sbi = 0; sbi < nblocks; ++sbi) {
    const uint8_t* bg = pg + sbi * 210;
    const uint8_t* bh = ph + sbi * 210;
    uint32_t scg[4], sch[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { scg[i] = lds32_a2(bg + 192 + 4 * i); sch[i] = lds32_a2(bh + 192 + 4 * i); }
    float usb[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) usb[nt][i] = 0.f;
#pragma unroll
    for (int ip = 0; ip < 2; ++ip) {
      uint32_t qlg[2][2], qhg[2], qlh[2][2], qhh[2];   // [s][half]
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        qlg[s][0] = lds32_a2(bg + 64 * ip + 16 * s + 4 * t);
        qlg[s][1] = lds32_a2(bg + 64 * ip + 32 + 16 * s + 4 * t);
        qhg[s] = lds32_a2(bg + 128 + 32 * ip + 16 * s + 4 * t);
        qlh[s][0] = lds32_a2(bh + 64 * ip + 16 * s + 4 * t);
        qlh[s][1] = lds32_a2(bh + 64 * ip + 32 + 16 * s + 4 * t);
        qhh[s] = lds32_a2(bh + 128 + 32 * ip + 16 * s + 4 * t);
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int b = b0 + sbi * 8 + 4 * ip + q4;
        int J[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) J[nt][i] = 0;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int gi = 8 * ip + 2 * q4 + s;
          const uint32_t ag = unpack6(qlg[s][q4 & 1], qhg[s], q4);
          const uint32_t ah = unpack6(qlh[s][q4 & 1], qhh[s], q4);
          const int sg = sext_byte(scg[gi >> 2], gi & 3);
          const int sh = sext_byte(sch[gi >> 2], gi & 3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t bb = *reinterpret_cast<const uint32_t*>(A.sA + (8 * nt + g) * A.a_stride + b * 32 + 16 * s + 4 * t);
            int D[4];
            mma_s8_k16(D, ag, ah, bb);
            J[nt][0] += D[0] * sg;
            J[nt][1] += D[1] * sg;
            J[nt][2] += D[2] * sh;
            J[nt][3] += D[3] * sh;
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float2 d8 = *reinterpret_cast<const float2*>(A.sD + b * 16 + 8 * nt + 2 * t);
          usb[nt][0] = fmaf((float)J[nt][0], d8.x, usb[nt][0]);
          usb[nt][1] = fmaf((float)J[nt][1], d8.y, usb[nt][1]);
          usb[nt][2] = fmaf((float)J[nt][2], d8.x, usb[nt][2]);
          usb[nt][3] = fmaf((float)J[nt][3], d8.y, usb[nt][3]);
        }
      }
    }
    const float dg = ld_h(bg + 208), dh = ld_h(bh + 208);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc[nt][0] = fmaf(dg, usb[nt][0], acc[nt][0]);
      acc[nt][1] = fmaf(dg, usb[nt][1], acc[nt][1]);
      acc[nt][2] = fmaf(dh, usb[nt][2], acc[nt][2]);
      acc[nt][3] = fmaf(dh, usb[nt][3], acc[nt][3]);
    }
  }
}

// ---------------------------------------------------------------------------------------------- kernel
// tensor-core consumers; NT = n-tiles of 8 tokens (MODE is always 0: the small-M path is gemv_rows_kernel)
template <int QT, int MODE, int NT, typename OutT>
__global__ void __launch_bounds__(cta_threads(MODE), 1) gemv_stream_kernel(const MmaParams p) {
  using F = Fmt<QT>;
  constexpr int NW = consumer_warps(MODE);
  constexpr int THREADS = cta_threads(MODE);
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + SMEM_HEADER - 8);
  volatile int* s_issued = reinterpret_cast<volatile int*>(smem + SMEM_HEADER - 32);   // stages issued, per producer warp
  uint32_t* s_grid = reinterpret_cast<uint32_t*>(smem + SMEM_HEADER);   // IQ3_S codebook (2 KB) when needed
  uint8_t* sA = smem + SMEM_HEADER + (QT == KQ_TYPE_IQ3_S ? 2048 : 0);
  float* sD = reinterpret_cast<float*>(sA + p.a_bytes);
  float* sZ = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sD) + p.d_bytes);
  uint8_t* ring = reinterpret_cast<uint8_t*>(sZ) + p.z_bytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  const int ks = blockIdx.x % p.ks;
  const int grp = blockIdx.x / p.ks, ngrp = gridDim.x / p.ks;
  const int rt0 = (int)((int64_t)grp * p.ntiles / ngrp), rt1 = (int)((int64_t)(grp + 1) * p.ntiles / ngrp);
  pdl_trigger();
  if (rt0 >= rt1) return;
  const int blk0 = (int)((int64_t)ks * p.nblk / p.ks), blk1 = (int)((int64_t)(ks + 1) * p.nblk / p.ks);
  const int nchunks = (blk1 - blk0 + p.cb - 1) / p.cb;
  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + MAX_STAGES), bar_act = smem_u32(bars + 2 * MAX_STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + 8 * s, NPROD); mbar_init(bar_empty + 8 * s, 1); }
    mbar_init(bar_act, 1);
    *s_abort = 0;
    for (int i = 0; i < NPROD; ++i) s_issued[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += THREADS) s_grid[i] = iq3s_expand(c_iq3s_codes_s[i], KQ_IQ3S_TOP);
  }
  __syncthreads();

  if (warp >= NW) {
    // ------------------------------------------------------------------ producers: warp pw fetches rows 4pw..4pw+3
    const int pw = warp - NW;
    const int k0 = blk0 * F::BLK, klen = (blk1 - blk0) * F::BLK;
    const int b32_0 = k0 >> 5, nb32 = klen >> 5;
    const int tt = p.m0 >> 4;
    constexpr int TOKCAP = 8 * NT;
    const int ntok = p.mcount < TOKCAP ? p.mcount : TOKCAP;
    const int mrow0 = p.m0;
    auto load_activations = [&]() {   // after pdl_wait(): the quantized activations come from the previous kernel
      if (lane == 0) {
        uint32_t total = (uint32_t)ntok * klen + (uint32_t)nb32 * 64u;
        if (p.zT != nullptr) total += (uint32_t)nb32 * p.zpb * 64u;
        mbar_expect_tx(bar_act, total);
      }
      __syncwarp();
      if (lane < ntok)
        bulk_g2s(smem_u32(sA + lane * p.a_stride), p.qs + (size_t)(mrow0 + lane) * p.kpad + k0, (uint32_t)klen, bar_act);
      if (lane == 16) bulk_g2s(smem_u32(sD), p.dT + ((size_t)tt * p.nb32tot + b32_0) * 16, (uint32_t)nb32 * 64u, bar_act);
      if (lane == 17 && p.zT != nullptr)
        bulk_g2s(smem_u32(sZ), p.zT + ((size_t)tt * p.nb32tot + b32_0) * p.zpb * 16, (uint32_t)nb32 * p.zpb * 64u, bar_act);
    };
    bool act_issued = false;

    int q = 0;
    bool ok = true;
    for (int rt = rt0; rt < rt1 && ok; ++rt) {
      const int row0 = rt * TILE_ROWS;
      for (int c = 0; c < nchunks && ok; ++c, ++q) {
        const int slot = q % S;
        if (q >= p.prefetch && pw == 0 && !act_issued) { pdl_wait(); load_activations(); act_issued = true; }
        if (q >= S) ok = mbar_wait(bar_empty + 8 * slot, (uint32_t)((q / S - 1) & 1), s_abort);
        if (!ok) break;
        const int blk_a = blk0 + c * p.cb;
        const int nb_c = (blk1 - blk_a) < p.cb ? (blk1 - blk_a) : p.cb;
        uint32_t bytes = 0;
        uintptr_t a0 = 0;
        const int rloc = pw * (TILE_ROWS / NPROD) + lane;
        const int row = row0 + rloc;
        if (lane < TILE_ROWS / NPROD && row < p.n) {
          const uintptr_t ga = (uintptr_t)(p.W + (size_t)row * p.rowbytes + (size_t)blk_a * F::BYTES);
          a0 = ga & ~(uintptr_t)15;
          bytes = (uint32_t)(((ga + (size_t)nb_c * F::BYTES + 15) & ~(uintptr_t)15) - a0);
        }
        uint32_t total = bytes;
#pragma unroll
        for (int mask = 16; mask > 0; mask >>= 1) total += __shfl_xor_sync(0xffffffffu, total, mask);
        if (lane == 0) {   // every producer warp arrives once per stage, with the bytes of its own rows (possibly 0)
          if (total) mbar_expect_tx(bar_full + 8 * slot, total); else mbar_arrive(bar_full + 8 * slot);
        }
        __syncwarp();
        if (bytes)
          bulk_g2s(smem_u32(ring + (size_t)slot * p.stage_bytes + (size_t)rloc * p.slot_stride), (const void*)a0, bytes,
                   bar_full + 8 * slot);
        if (lane == 0) { __threadfence_block(); s_issued[pw] = q + 1; }   // after the expect_tx of this stage
      }
    }
    if (pw == 0 && !act_issued) { pdl_wait(); load_activations(); act_issued = true; }
    // copies still in flight must land before the CTA may exit
    const int first = q > S ? q - S : 0;
    for (int qq = first; qq < q; ++qq) mbar_wait(bar_full + 8 * (qq % S), (uint32_t)((qq / S) & 1), s_abort);
    if (!ok && lane == 0) atomicExch(p.status, 1);
    return;
  }

  // -------------------------------------------------------------------- consumers
  if (!mbar_wait(bar_act, 0, s_abort)) { if (lane == 0) atomicExch(p.status, 2); return; }
  ActView A{sA, p.a_stride, sD, sZ};
  OutT* y = reinterpret_cast<OutT*>(p.y);
  const int tok0 = p.m0 & 15;                     // first token of this pass inside its 16-token tile

  if constexpr (MODE == 0) {
    // ---- a warp owns whole tiles
    const int g = lane >> 2, t = lane & 3;
    for (int idx = warp; rt0 + idx < rt1; idx += NW) {
      const int rt = rt0 + idx, row0 = rt * TILE_ROWS;
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
      const size_t rbg = (size_t)(row0 + g) * p.rowbytes, rbh = (size_t)(row0 + g + 8) * p.rowbytes;
      for (int c = 0; c < nchunks; ++c) {
        const int q = idx * nchunks + c, slot = q % S;
        auto issued = [&]() { return s_issued[0] > q && s_issued[1] > q && s_issued[2] > q && s_issued[3] > q; };
        if (!issued()) {   // not issued yet: the slot's barrier may still show an older generation
          const long long t0 = clock64();
          while (!issued()) {
            if (*s_abort || clock64() - t0 > WAIT_LIMIT) { *s_abort = 1; if (lane == 0) atomicExch(p.status, 4); return; }
          }
        }
        if (!mbar_wait(bar_full + 8 * slot, (uint32_t)((q / S) & 1), s_abort)) { if (lane == 0) atomicExch(p.status, 3); return; }
        const int blk_a = blk0 + c * p.cb;
        const int nb_c = (blk1 - blk_a) < p.cb ? (blk1 - blk_a) : p.cb;
        const uint8_t* st = ring + (size_t)slot * p.stage_bytes;
        const uint32_t offg = (uint32_t)(((uintptr_t)p.W + rbg + (size_t)blk_a * F::BYTES) & 15);
        const uint32_t offh = (uint32_t)(((uintptr_t)p.W + rbh + (size_t)blk_a * F::BYTES) & 15);
        const uint8_t* pg = st + (size_t)g * p.slot_stride + offg;
        const uint8_t* ph = st + (size_t)(g + 8) * p.slot_stride + offh;
        const int b0 = (blk_a - blk0) * (F::BLK / 32);
        if constexpr (QT == KQ_TYPE_Q4_K) chunk_q4k<NT>(pg, ph, nb_c, b0, A, g, t, acc);
        if constexpr (QT == KQ_TYPE_Q6_K) chunk_q6k<NT>(pg, ph, nb_c, b0, A, g, t, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
      }
      // lane holds rows g (i=0,1) and g+8 (i=2,3), tokens 8nt+2t (+1)
      if (p.ks == 1) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = row0 + g + ((i >> 1) << 3), tl = 8 * nt + 2 * t + (i & 1);
            if (row < p.n && tl < p.mcount) y[(size_t)(p.m0 + tl) * p.stride_y + row] = from_f32<OutT>(acc[nt][i]);
          }
      } else {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = row0 + g + ((i >> 1) << 3), tl = 8 * nt + 2 * t + (i & 1);
            if (row < p.n && tl < p.mcount) __stcg(p.part + ((size_t)ks * 16 + tl) * p.n + row, acc[nt][i]);
          }
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(p.cnt + rt, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == p.ks - 1) {   // every split of this tile has published: add them in split order
          __threadfence();
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int row = row0 + g + ((i >> 1) << 3), tl = 8 * nt + 2 * t + (i & 1);
              if (row < p.n && tl < p.mcount) {
                float sum = 0.f;
                for (int sp = 0; sp < p.ks; ++sp) sum += __ldcg(p.part + ((size_t)sp * 16 + tl) * p.n + row);
                y[(size_t)(p.m0 + tl) * p.stride_y + row] = from_f32<OutT>(sum);
              }
            }
          if (lane == 0) p.cnt[rt] = 0;   // ready for the next launch on this scratch
        }
      }
    }
  }
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
  if (p.x != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && p.m0 == 0) *p.status = 0;   // no quantizer launch clears it
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
        const uintptr_t ga = (uintptr_t)(p.W + (size_t)ra * p.rowbytes);
        const uintptr_t ge = (uintptr_t)(p.W + (size_t)rb * p.rowbytes);
        const uintptr_t a0 = ga & ~(uintptr_t)15;
        const uint32_t bytes = (uint32_t)(((ge + 15) & ~(uintptr_t)15) - a0);
        mbar_expect_tx(bar_full + 8 * slot, bytes);
        bulk_g2s(smem_u32(ring + (size_t)slot * p.stage_bytes), (const void*)a0, bytes, bar_full + 8 * slot);
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
  }
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
        if constexpr (NG == 1) {
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

// ---------------------------------------------------------------------------------------------- host
struct Config {
  int ks, cb, stages, slot_stride, stage_bytes, a_stride, a_bytes, d_bytes, z_bytes, smem, grid;
};
struct RowConfig {
  int rows_per_stage, stages, stage_bytes, a_stride, a_bytes, d_bytes, z_bytes, smem, grid;
};

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

int z_per_block(int type) {
  return (type == KQ_TYPE_Q2_K) ? 2 : ((type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q4_0) ? 1 : 0);
}

constexpr int SMEM_LIMIT = 227 * 1024;

// tensor-core kernel: mtok = token rows of the activation slice kept in shared memory (8 or 16)
bool make_config(int type, int64_t n, int64_t k, int mtok, Config& c) {
  int blk, bytes;
  if (!type_geometry(type, &blk, &bytes)) return false;
  const int nblk = (int)(k / blk);
  const int ntiles = (int)((n + 15) / 16);
  const int sms = sm_count();
  const int zpb = z_per_block(type);
  const int header = SMEM_HEADER + (type == KQ_TYPE_IQ3_S ? 2048 : 0);
  double best = 1e30;
  bool found = false;
  for (int ks = 1; ks <= 4; ks *= 2) {
    if (nblk < ks) break;
    const int grid = sms / ks * ks;
    const int ngrp = grid / ks;
    const int klen = ((nblk + ks - 1) / ks) * blk;
    // chunk = row segment of about 2 KB (>= ~1 KB keeps the copy engine at HBM speed), evenly dividing the split
    const int bps = (nblk + ks - 1) / ks;
    int cb_target = 2048 / bytes;
    if (cb_target < 1) cb_target = 1;
    const int nch = (bps + cb_target - 1) / cb_target;
    const int cb = (bps + nch - 1) / nch;
    const int resid = type == KQ_TYPE_Q4_K ? 32 : 16;   // row-slot stride mod 128: spreads the 16 rows over the banks
    int slot = ((cb * bytes + 16 + 15) / 16) * 16;
    while (slot % 128 != resid) slot += 16;
    const int stage_bytes = 16 * slot;
    const int a_stride = klen + 32;
    const int a_bytes = (mtok * a_stride + 127) / 128 * 128;
    const int d_bytes = ((klen / 32) * 64 + 127) / 128 * 128;
    const int z_bytes = ((klen / 32) * 64 * zpb + 127) / 128 * 128;
    const int fixed = header + a_bytes + d_bytes + z_bytes;
    int stages = (SMEM_LIMIT - fixed) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 3) continue;
    const int per = (ntiles + ngrp - 1) / ngrp;
    const double cost = (double)per / ks + 0.02 * (ks - 1);   // tiles per CTA x work per tile, small bias to fewer splits
    if (cost < best - 1e-9) {
      best = cost; found = true;
      c.ks = ks; c.grid = grid; c.a_stride = a_stride; c.a_bytes = a_bytes; c.d_bytes = d_bytes; c.z_bytes = z_bytes;
      c.cb = cb; c.slot_stride = slot; c.stage_bytes = stage_bytes;
      c.stages = stages; c.smem = fixed + stages * stage_bytes;
    }
  }
  return found;
}

// row-streaming kernel: whole rows per stage, the full K of `mt` tokens resident in shared memory
bool make_row_config(int type, int64_t n, int64_t k, int mt, bool pair, RowConfig& c) {
  int blk, bytes;
  if (!type_geometry(type, &blk, &bytes)) return false;
  const int64_t rowbytes = k / blk * bytes;
  const int zpb = z_per_block(type);
  int R = (int)(16384 / rowbytes);
  if (R < 1) R = 1;
  if (R > 16) R = 16;
  if (pair) R = R < 2 ? 2 : (R & ~1);   // a warp's two rows never straddle stages
  c.rows_per_stage = R;
  c.stage_bytes = (int)((R * rowbytes + 32 + 127) / 128 * 128);
  const int64_t kpad = (k + 511) / 512 * 512;
  const bool zr = type == KQ_TYPE_Q2_K || type == KQ_TYPE_Q4_K || (pair && type == KQ_TYPE_Q6_K);
  c.a_stride = pair ? (int)(k / 64) * 80 + 16 : (int)k + 32;
  c.a_bytes = (mt * c.a_stride + 127) / 128 * 128;
  c.d_bytes = (int)((mt * (kpad / 32) * 4 + 127) / 128 * 128);
  c.z_bytes = zr ? (int)((mt * (kpad / 32) * 4 * (type == KQ_TYPE_Q4_K ? 1 : 2) + 127) / 128 * 128) : 0;
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

template <int QT, int NT, typename OutT>
int launch_tc(const MmaParams& p, const Config& c, cudaStream_t st) {
  auto kern = gemv_stream_kernel<QT, 0, NT, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    attr_set = true;
  }
  KQ_CUDA_TRY(launch_pdl(kern, dim3(c.grid), dim3(cta_threads(0)), (size_t)c.smem, st, options().pdl != 0, p));
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT, int MT, bool PAIR, typename OutT>
int launch_rows(const RowParams& p, const RowConfig& c, cudaStream_t st) {
  auto kern = gemv_rows_kernel<QT, MT, PAIR, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    attr_set = true;
  }
  KQ_CUDA_TRY(launch_pdl(kern, dim3(c.grid), dim3(ROW_THREADS), (size_t)c.smem, st, options().pdl != 0, p));
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT, typename OutT>
int launch_tc_nt(const MmaParams& p, const Config& c, int nt, cudaStream_t st) {
  if constexpr (QT == KQ_TYPE_Q4_K || QT == KQ_TYPE_Q6_K) {
    return nt == 2 ? launch_tc<QT, 2, OutT>(p, c, st) : launch_tc<QT, 1, OutT>(p, c, st);
  } else {
    set_error("tensor-core GEMV: type not covered");
    return KQ_EUNSUPPORTED;
  }
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
int launch_typed(const MmaParams* pt, const Config* ct, const RowParams* pr, const RowConfig* cr, int nt, int y_dtype,
                 cudaStream_t st) {
  switch (y_dtype) {
    case KQ_F32: return pt ? launch_tc_nt<QT, float>(*pt, *ct, nt, st) : launch_rows_mt<QT, float>(*pr, *cr, nt, st);
    case KQ_F16: return pt ? launch_tc_nt<QT, __half>(*pt, *ct, nt, st) : launch_rows_mt<QT, __half>(*pr, *cr, nt, st);
    case KQ_BF16: return pt ? launch_tc_nt<QT, __nv_bfloat16>(*pt, *ct, nt, st) : launch_rows_mt<QT, __nv_bfloat16>(*pr, *cr, nt, st);
  }
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace

// The streaming kernels fetch weights in 16-byte units and (Q4_K tensor-core mode) read 64-bit words, so they
// need a 16-byte aligned weight pointer; anything else goes to the general dp4a kernel.
bool gemv_mma_supported(const void* W, int type, int64_t n, int64_t k) {
  if ((uintptr_t)W % 16) return false;
  RowConfig c;
  return make_row_config(type, n, k, 1, false, c);
}

// impl: 0 = choose by m, 2 = tensor cores wherever the type has them, 3 = row-streaming dp4a
// Smallest token count that goes to the shared-stage mma kernel in auto mode.  Q4_0's 18-byte blocks decode slowly
// there (row-streaming kernel up to 8 tokens).  Q6_K's row-streaming consumer tops out near 3 TB/s, the mma kernel
// near 4.2 TB/s, so whenever it needs no K split (K up to about 8K) the mma kernel takes 1-2 tokens as well: 27.2 ->
// 21.0 us on 17408x5120, 352 -> 246 us on a 248320x5120 LM head; with a K split (5120x17408) the row kernel stays ahead.
static int tile_min_tokens(int type, int64_t n, int64_t k) {
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

// fuse_x != nullptr (only with gemv_rows_only): the activations have NOT been quantized into P; the kernel reads them raw
int launch_gemv_mma(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m, void* y, int y_dtype,
                    int64_t stride_y, bool mmq, cudaStream_t st, const void* fuse_x, int x_dtype, int64_t stride_x) {
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  const int impl = options().gemv_impl;
  const bool has_tc = (type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q6_K);
  if (impl == 2 && !has_tc) { set_error("tensor-core GEMV: type %d not covered", type); return KQ_EUNSUPPORTED; }
  const float* zT = nullptr;
  if (type == KQ_TYPE_Q4_K) zT = mmq ? P.zs8 : P.z32;
  if (type == KQ_TYPE_Q4_0) zT = P.zs8;
  if (type == KQ_TYPE_Q2_K) zT = P.z16;
  const int zpb = z_per_block(type) ? z_per_block(type) : 1;
  int64_t m0 = 0;
  while (m0 < m) {
    const int64_t left = m - m0;
    const bool tile_start = (m0 % 16) == 0;
    int rc, mcount;
    Config c;
    // the tcgen05 kernel runs on request only (impl 5): its 144-byte weight rows keep the copy engine request-bound
    if (tile_start && impl == 5 && gemv_tc5_supported(W, type, n, k)) {
      mcount = (int)(left < 16 ? left : 16);
      rc = launch_gemv_tc5(W, type, n, k, P, m, m0, mcount, y, y_dtype, stride_y, mmq, st);
      if (rc) return rc;
      m0 += mcount;
      continue;
    }
    if (impl == 5) { set_error("tcgen05 GEMV: type/shape not covered"); return KQ_EUNSUPPORTED; }
    // 3..16 tokens of Q4_K / Q6_K: the shared-stage mma kernel (all warps of a CTA on every stage of 8 rows)
    const int tile_min = tile_min_tokens(type, n, k);
    if (tile_start && (impl == 6 || (impl == 0 && left >= tile_min)) &&
        gemv_tile_supported(W, type, n, k, (int)(left < 16 ? left : 16))) {
      mcount = (int)(left < 16 ? left : 16);
      rc = launch_gemv_tile(W, type, n, k, P, m0, mcount, y, y_dtype, stride_y, mmq, st);
      if (rc) return rc;
      m0 += mcount;
      continue;
    }
    if (impl == 6) { set_error("tile GEMV: type/shape not covered"); return KQ_EUNSUPPORTED; }
    if (has_tc && tile_start && impl != 3 && impl != 4 && (impl == 2 || left >= options().tc_min_m) &&
        make_config(type, n, k, left > 8 ? 16 : 8, c)) {
      mcount = (int)(left < 16 ? left : 16);
      const int nt = mcount > 8 ? 2 : 1;
      MmaParams p;
      p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.n = (int)n; p.nblk = (int)(k / blk); p.ks = c.ks;
      p.ntiles = (int)((n + 15) / 16); p.cb = c.cb; p.stages = c.stages; p.slot_stride = c.slot_stride;
      p.stage_bytes = c.stage_bytes; p.a_stride = c.a_stride; p.a_bytes = c.a_bytes; p.d_bytes = c.d_bytes;
      p.z_bytes = c.z_bytes; p.qs = P.qs; p.dT = P.dT; p.kpad = (int)P.kpad; p.nb32tot = (int)(P.kpad / 32);
      p.zT = zT; p.zpb = zpb;
      p.prefetch = options().pdl < c.stages ? options().pdl : c.stages;
      p.m0 = (int)m0; p.mcount = mcount; p.y = y; p.stride_y = stride_y; p.part = P.part; p.cnt = P.cnt; p.status = P.status;
      rc = type == KQ_TYPE_Q4_K ? launch_typed<KQ_TYPE_Q4_K>(&p, &c, nullptr, nullptr, nt, y_dtype, st)
                                : launch_typed<KQ_TYPE_Q6_K>(&p, &c, nullptr, nullptr, nt, y_dtype, st);
    } else {
      if (impl == 2) { set_error("tensor-core GEMV: no configuration for this shape"); return KQ_EUNSUPPORTED; }
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
      if (type == KQ_TYPE_Q4_0 || (type == KQ_TYPE_Q4_K && mmq)) p.zmode = 1;
      else if (type == KQ_TYPE_Q4_K) { p.zmode = 2; p.zr = P.z32r; }
      else if (type == KQ_TYPE_Q2_K) { p.zmode = 3; p.zr = P.z16r; }
      else if (type == KQ_TYPE_Q6_K && pair) { p.zmode = 3; p.zr = P.z16r; p.zpb = 2; }   // -32 offset via group sums
      p.prefetch = options().pdl < rcg.stages ? options().pdl : rcg.stages;
      p.m0 = (int)m0; p.mcount = mcount; p.y = y; p.stride_y = stride_y; p.status = P.status;
      p.x = fuse_x; p.x_dtype = x_dtype; p.stride_x = stride_x;
      switch (type) {
        case KQ_TYPE_Q4_0: rc = launch_typed<KQ_TYPE_Q4_0>(nullptr, nullptr, &p, &rcg, mt, y_dtype, st); break;
        case KQ_TYPE_Q8_0: rc = launch_typed<KQ_TYPE_Q8_0>(nullptr, nullptr, &p, &rcg, mt, y_dtype, st); break;
        case KQ_TYPE_Q2_K: rc = launch_typed<KQ_TYPE_Q2_K>(nullptr, nullptr, &p, &rcg, mt, y_dtype, st); break;
        case KQ_TYPE_Q4_K: rc = launch_typed<KQ_TYPE_Q4_K>(nullptr, nullptr, &p, &rcg, mt, y_dtype, st); break;
        case KQ_TYPE_Q6_K: rc = launch_typed<KQ_TYPE_Q6_K>(nullptr, nullptr, &p, &rcg, mt, y_dtype, st); break;
        default: rc = launch_typed<KQ_TYPE_IQ3_S>(nullptr, nullptr, &p, &rcg, mt, y_dtype, st); break;
      }
    }
    if (rc) return rc;
    m0 += mcount;
  }
  return KQ_OK;
}

}  // namespace kq
