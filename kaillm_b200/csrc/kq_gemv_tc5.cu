// Decode GEMV on the 5th-generation tensor cores (tcgen05 kind::i8, TMEM), Q4_K, 5 <= M <= 16 tokens per pass.
//
// Why: with more than ~4 tokens the integer dots of a GEMV cost more issue slots than the HBM stream leaves
// (dp4a and mma.sync both need per-lane fragment handling).  Here a thread only unpacks nibbles and applies
// scales; the dots run as UMMA instructions issued by one thread.
//
//   work unit   (128-row tile, 256-weight super-block).  Units are linearised tile-major and cut into 148 equal
//               contiguous ranges, one per CTA (stream-K): every SM streams the same number of bytes whatever
//               the shape.  A range that covers only part of a tile's K ends in a partial sum; the partials of a
//               tile are added in CTA order by the last contributor to arrive (deterministic), full tiles are
//               stored directly.
//   weights     one TMA tiled load per unit: box = 128 rows x 144 bytes (a single copy-engine request of 18 KB;
//               per-row segment copies would be request-rate bound), 6-deep ring.
//   activations the int8 codes of the CTA's K window, 16 token rows (rows past m read as zero), TMA tiled loads
//               with 128-byte swizzle = the K-major B operand; scale tables [block][16 tokens] by bulk copy.
//   8 warps     thread = (row, half of the super-block): unpack 4 sub-blocks (64 nibble bytes) to int8, write them
//               to TMEM (tcgen05.st) as the A operand; later read the 4 x 16 int32 dots of those sub-blocks back
//               (tcgen05.ld) and fold them into 16 fp32 accumulators with the row's 6-bit scales / mins and the
//               tokens' d8 / min-term tables.  Software-pipelined: unpack(u+1) is issued before epilogue(u).
//   warp 8      TMA producer (one lane); warp 9: MMA issuer (one lane): per unit 8 x tcgen05.mma.kind::i8
//               (M=128, N=16, K=32), one per sub-block, each into its own 16 TMEM columns (no accumulation across
//               sub-blocks: every 32-block has its own activation scale), then tcgen05.commit.
//   TMEM        A: 2 x 64 columns, D: 2 x 128 columns.
//
// Integer dots are exact; the fp32 combine follows vec_dot_q4_K_q8_1 (vecdotq.cuh:328-379 of the reference).
// All waits are bounded (status word, abort flag, TMEM released before return).
#include <cuda.h>

#include "kq_common.cuh"

namespace kq {
namespace {

constexpr int T5_ROWS = 128;
constexpr int T5_NTOK = 16;
constexpr int T5_WSTAGES = 6;
constexpr int T5_WBYTES = T5_ROWS * 144;        // 18432
constexpr int T5_DQ_WARPS = 8;
constexpr int T5_THREADS = (T5_DQ_WARPS + 2) * 32;
constexpr uint32_t T5_TMEM_COLS = 512;
constexpr uint32_t T5_TMEM_D = 0;               // 2 x 128 columns
constexpr uint32_t T5_TMEM_A = 256;             // 2 x 64 columns
constexpr long long T5_WAIT_LIMIT = 1ll << 27;
constexpr uint32_t T5_MAGIC_I = 0x4B400000u;
constexpr float T5_MAGIC_F = 12582912.0f;

struct Tc5Params {
  int n, nsb;                 // rows, super-blocks per row
  int ntiles;
  int64_t units;              // ntiles * nsb
  int m0, mcount;
  int asb_cap;                // super-blocks of activations the shared-memory window can hold
  const float* dT;            // [tt][nb32][16]
  const float* zT;            // [tt][nb32][16]
  int nb32tot;
  void* y;
  int64_t stride_y;
  float* part;                // [slot][16][n]
  int* cnt;                   // per tile
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
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > T5_WAIT_LIMIT) { *abort_flag = 1; return false; }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&a)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]),
        "r"(a[9]), "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(a[16]), "r"(a[17]), "r"(a[18]),
        "r"(a[19]), "r"(a[20]), "r"(a[21]), "r"(a[22]), "r"(a[23]), "r"(a[24]), "r"(a[25]), "r"(a[26]), "r"(a[27]), "r"(a[28]),
        "r"(a[29]), "r"(a[30]), "r"(a[31]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// loads without the wait: several can be in flight before one tcgen05.wait::ld
__device__ __forceinline__ void tmem_ld4_nw(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8_nw(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16_nw(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
template <int NT> __device__ __forceinline__ void tmem_ld_nt(uint32_t taddr, uint32_t* r) {
  if constexpr (NT == 4) tmem_ld4_nw(taddr, r);
  else if constexpr (NT == 8) tmem_ld8_nw(taddr, r);
  else tmem_ld16_nw(taddr, r);
}

// first unit of CTA c when `units` are cut into `g` contiguous ranges
__device__ __forceinline__ int64_t range_lo(int64_t c, int64_t units, int64_t g) { return c * units / g; }
// CTA that owns unit u
__device__ __forceinline__ int owner_of(int64_t u, int64_t units, int g) {
  int c = (int)(((u + 1) * g - 1) / units);   // first guess, then settle on lo(c) <= u < lo(c+1)
  if (c >= g) c = g - 1;
  while (c > 0 && range_lo(c, units, g) > u) --c;
  while (c + 1 < g && range_lo(c + 1, units, g) <= u) ++c;
  return c;
}

// NT: token columns the epilogue reads back and accumulates (4, 8 or 16 >= mcount)
template <int NT, typename OutT>
__global__ void __launch_bounds__(T5_THREADS, 1)
gemv_tc5_q4k_kernel(const Tc5Params p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap qmap) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // layout: [W ring 6 x 18 KB][activation atoms asb_cap*2 x 2 KB][d8 table][z table][barriers]
  uint8_t* sW = smem;
  uint8_t* sQ = sW + T5_WSTAGES * T5_WBYTES;                                   // 1024-aligned: 110592 = 108 * 1024
  float* sD = reinterpret_cast<float*>(sQ + (size_t)p.asb_cap * 2 * 2048);
  float* sZ = sD + (size_t)p.asb_cap * 8 * 16;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sZ + (size_t)p.asb_cap * 8 * 16);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 25);
  volatile int* s_last = reinterpret_cast<volatile int*>(bars + 26);
  const uint32_t bar_wfull = smem_u32(bars), bar_wempty = smem_u32(bars + 6), bar_afull = smem_u32(bars + 12),
                 bar_dfull = smem_u32(bars + 14), bar_act = smem_u32(bars + 16), bar_dfree = smem_u32(bars + 18),
                 bar_sync128 = smem_u32(bars + 20);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x;
  const int64_t u_lo = range_lo(blockIdx.x, p.units, G), u_hi = range_lo(blockIdx.x + 1, p.units, G);
  const int nunits = (int)(u_hi - u_lo);
  if (nunits <= 0) return;
  const int nsb = p.nsb;
  // activation window: the whole K if the range covers at least one tile's worth of units, else the nunits
  // super-blocks it touches (contiguous modulo nsb).  Window slot of super-block sb = (sb - w0) mod nsb.
  const int sb_first = (int)(u_lo % nsb);
  const bool full_k = nunits >= nsb;
  const int w0 = full_k ? 0 : sb_first;
  const int wlen = full_k ? nsb : nunits;

  if (tid == 0) {
    for (int i = 0; i < T5_WSTAGES; ++i) { mbar_init(bar_wfull + 8 * i, 1); mbar_init(bar_wempty + 8 * i, T5_DQ_WARPS); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_afull + 8 * i, 4);      // the four unpacking warps
      mbar_init(bar_dfull + 8 * i, 1);      // tcgen05.commit
      mbar_init(bar_dfree + 8 * i, 4);      // the four epilogue warps have read the accumulators
    }
    mbar_init(bar_act, 1);
    mbar_init(bar_sync128, 128);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(T5_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tbase = *tmem_slot;
  const int rloc = (warp & 3) * 32 + lane;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

  if (warp == T5_DQ_WARPS) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int tt = p.m0 >> 4;
      mbar_expect_tx(bar_act, (uint32_t)wlen * (2 * 2048 + 2 * 8 * 64));
      for (int s = 0; s < wlen; ++s) {
        const int sb = (w0 + s) % nsb;
        tma_load_2d(smem_u32(sQ + (size_t)(2 * s) * 2048), &qmap, sb * 256, p.m0, bar_act);
        tma_load_2d(smem_u32(sQ + (size_t)(2 * s + 1) * 2048), &qmap, sb * 256 + 128, p.m0, bar_act);
        bulk_g2s(smem_u32(sD + (size_t)s * 8 * 16), p.dT + ((size_t)tt * p.nb32tot + sb * 8) * 16, 8 * 64, bar_act);
        bulk_g2s(smem_u32(sZ + (size_t)s * 8 * 16), p.zT + ((size_t)tt * p.nb32tot + sb * 8) * 16, 8 * 64, bar_act);
      }
      bool ok = true;
      for (int i = 0; i < nunits && ok; ++i) {
        const int slot = i % T5_WSTAGES, fill = i / T5_WSTAGES;
        if (fill > 0) ok = mbar_wait(bar_wempty + 8 * slot, (uint32_t)((fill - 1) & 1), s_abort);
        if (!ok) break;
        const int64_t u = u_lo + i;
        const int tile = (int)(u / nsb), sb = (int)(u % nsb);
        mbar_expect_tx(bar_wfull + 8 * slot, T5_WBYTES);
        tma_load_2d(smem_u32(sW + (size_t)slot * T5_WBYTES), &wmap, sb * 36, tile * T5_ROWS, bar_wfull + 8 * slot);
      }
      const int first = nunits > T5_WSTAGES ? nunits - T5_WSTAGES : 0;   // loads in flight must land before exit
      for (int i = first; i < nunits; ++i) mbar_wait(bar_wfull + 8 * (i % T5_WSTAGES), (uint32_t)((i / T5_WSTAGES) & 1), s_abort);
    }
  } else if (warp == T5_DQ_WARPS + 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // D = s32, A = u8 (nibbles 0..15), B = s8, both K-major, N = 16, M = 128
      const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(T5_NTOK >> 3) << 17) | ((uint32_t)(T5_ROWS >> 4) << 24);
      bool ok = mbar_wait(bar_act, 0, s_abort);
      for (int i = 0; i < nunits && ok; ++i) {
        const int buf = i & 1;
        ok = mbar_wait(bar_afull + 8 * buf, (uint32_t)((i >> 1) & 1), s_abort);
        if (ok && i >= 2) ok = mbar_wait(bar_dfree + 8 * buf, (uint32_t)(((i >> 1) - 1) & 1), s_abort);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int sb = (int)((u_lo + i) % nsb);
        const int ws = (sb - w0 + nsb) % nsb;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t baddr = smem_u32(sQ + (size_t)(2 * ws + (j >> 2)) * 2048);
          const uint64_t bdesc = ((uint64_t)((baddr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
                                  (1ull << 46) | (2ull << 61)) + (uint64_t)(((j & 3) * 32) >> 4);
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
              ::"r"(tbase + T5_TMEM_D + buf * 128 + j * 16), "r"(tbase + T5_TMEM_A + buf * 64 + j * 8), "l"(bdesc), "r"(idesc), "r"(0u)
              : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_dfull + 8 * buf) : "memory");
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ unpackers: thread = row
    bool ok = true;
    for (int i = 0; i < nunits && ok; ++i) {
      const int slot = i % T5_WSTAGES, buf = i & 1;
      ok = mbar_wait(bar_wfull + 8 * slot, (uint32_t)((i / T5_WSTAGES) & 1), s_abort);
      if (!ok) break;
      const uint8_t* bp = sW + (size_t)slot * T5_WBYTES + (size_t)rloc * 144;
      uint32_t a[64];
#pragma unroll
      for (int il = 0; il < 4; ++il) {     // nibble run il: sub-blocks 2il (low nibbles) and 2il+1 (high nibbles)
        const uint4 w0v = *reinterpret_cast<const uint4*>(bp + 16 + 32 * il);
        const uint4 w1v = *reinterpret_cast<const uint4*>(bp + 32 + 32 * il);
        const uint32_t wq[8] = {w0v.x, w0v.y, w0v.z, w0v.w, w1v.x, w1v.y, w1v.z, w1v.w};
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          a[16 * il + r] = wq[r] & 0x0F0F0F0Fu;
          a[16 * il + 8 + r] = (wq[r] >> 4) & 0x0F0F0F0Fu;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_wempty + 8 * slot);
      // A[buf] is free once the MMAs of unit i-2 have completed (the commit that also publishes their accumulators)
      if (i >= 2) ok = mbar_wait(bar_dfull + 8 * buf, (uint32_t)(((i >> 1) - 1) & 1), s_abort);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t (&alo)[32] = *reinterpret_cast<const uint32_t (*)[32]>(&a[0]);
      const uint32_t (&ahi)[32] = *reinterpret_cast<const uint32_t (*)[32]>(&a[32]);
      tmem_st32(tbase + T5_TMEM_A + lane_base + buf * 64, alo);
      tmem_st32(tbase + T5_TMEM_A + lane_base + buf * 64 + 32, ahi);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_afull + 8 * buf);
    }
  } else {
    // ------------------------------------------------------------------ epilogue: thread = row
    OutT* y = reinterpret_cast<OutT*>(p.y);
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.f;
    bool ok = mbar_wait(bar_act, 0, s_abort);
    uint32_t ph128 = 0;
    int seg_units = 0;
    for (int i = 0; i < nunits && ok; ++i) {
      const int slot = i % T5_WSTAGES, buf = i & 1;
      ok = mbar_wait(bar_wfull + 8 * slot, (uint32_t)((i / T5_WSTAGES) & 1), s_abort);
      if (!ok) break;
      const uint4 hdr = *reinterpret_cast<const uint4*>(sW + (size_t)slot * T5_WBYTES + (size_t)rloc * 144);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_wempty + 8 * slot);
      // 6-bit scales / mins as bytes: word 0 = sub-blocks 0-3, word 1 = 4-7
      const uint32_t scw[2] = {hdr.y & 0x3F3F3F3Fu, (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u)};
      const uint32_t mnw[2] = {hdr.z & 0x3F3F3F3Fu, ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u)};
      const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
      ok = mbar_wait(bar_dfull + 8 * buf, (uint32_t)((i >> 1) & 1), s_abort);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int sb = (int)((u_lo + i) % nsb);
      const int ws = (sb - w0 + nsb) % nsb;
      float u[NT], um[NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) { u[t] = 0.f; um[t] = 0.f; }
      // read the accumulators back in groups of GJ sub-blocks (all loads of a group in flight before one wait)
      constexpr int GJ = NT == 16 ? 4 : 8;
#pragma unroll
      for (int j0 = 0; j0 < 8; j0 += GJ) {
        uint32_t d[GJ][NT];
#pragma unroll
        for (int jj = 0; jj < GJ; ++jj) tmem_ld_nt<NT>(tbase + T5_TMEM_D + lane_base + buf * 128 + (j0 + jj) * 16, d[jj]);
        tmem_wait_ld();
        if (j0 + GJ == 8) {   // all accumulators of this unit are in registers: the MMA warp may overwrite D[buf]
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_dfree + 8 * buf);
        }
#pragma unroll
        for (int jj = 0; jj < GJ; ++jj) {
          const int j = j0 + jj;
          const int sc = (int)((scw[j >> 2] >> (8 * (j & 3))) & 0xFFu);
          const float mn = (float)((mnw[j >> 2] >> (8 * (j & 3))) & 0xFFu);
          const float4* d8p = reinterpret_cast<const float4*>(sD + ((size_t)ws * 8 + j) * 16);
          const float4* zp = reinterpret_cast<const float4*>(sZ + ((size_t)ws * 8 + j) * 16);
#pragma unroll
          for (int q = 0; q < NT / 4; ++q) {
            const float4 d8 = d8p[q], z = zp[q];
            const float dd[4] = {d8.x, d8.y, d8.z, d8.w}, zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int t = 4 * q + e;
              // |dot * sc| <= 60960 * 63 < 2^22: exact int -> float through the 1.5*2^23 constant
              const float f = __int_as_float((int)d[jj][t] * sc + (int)T5_MAGIC_I) - T5_MAGIC_F;
              u[t] = fmaf(f, dd[e], u[t]);
              um[t] = fmaf(mn, zz[e], um[t]);
            }
          }
        }
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) acc[t] += dm.x * u[t] - dm.y * um[t];
      ++seg_units;
      const int64_t uu = u_lo + i;
      if (((uu + 1) % nsb) == 0 || i + 1 == nunits) {
        // ---- end of this CTA's segment of the tile: store, or publish a partial and let the last contributor add
        const int tile = (int)(uu / nsb);
        const int row = tile * T5_ROWS + rloc;
        if (seg_units == nsb) {
          if (row < p.n) {
#pragma unroll
            for (int t = 0; t < NT; ++t)
              if (t < p.mcount) y[(size_t)(p.m0 + t) * p.stride_y + row] = from_f32<OutT>(acc[t]);
          }
        } else {
          const int64_t t_lo = (int64_t)tile * nsb;
          const int c_first = owner_of(t_lo, p.units, G), c_last = owner_of(t_lo + nsb - 1, p.units, G);
          const int pslot = (int)blockIdx.x - c_first;
          if (row < p.n) {
#pragma unroll
            for (int t = 0; t < NT; ++t)
              if (t < p.mcount) __stcg(p.part + ((size_t)pslot * 16 + t) * p.n + row, acc[t]);
          }
          __threadfence();
          // bounded rendezvous of the 128 epilogue threads (an mbarrier, not bar.sync: a thread that gave up
          // must not strand the others)
          mbar_arrive(bar_sync128);
          ok = mbar_wait(bar_sync128, ph128, s_abort); ph128 ^= 1u;
          if (!ok) break;
          if (rloc == 0) {
            const int old = atomicAdd(p.cnt + tile, 1);
            *s_last = (old == c_last - c_first) ? 1 : 0;
          }
          mbar_arrive(bar_sync128);
          ok = mbar_wait(bar_sync128, ph128, s_abort); ph128 ^= 1u;
          if (!ok) break;
          const bool last = *s_last != 0;
          mbar_arrive(bar_sync128);                     // everyone has read s_last before it can be rewritten
          ok = mbar_wait(bar_sync128, ph128, s_abort); ph128 ^= 1u;
          if (!ok) break;
          if (last) {
            __threadfence();
            if (row < p.n) {
              const int ncontrib = c_last - c_first + 1;
#pragma unroll
              for (int t = 0; t < NT; ++t) {
                if (t < p.mcount) {
                  float sum = 0.f;
                  for (int sp = 0; sp < ncontrib; ++sp) sum += __ldcg(p.part + ((size_t)sp * 16 + t) * p.n + row);
                  y[(size_t)(p.m0 + t) * p.stride_y + row] = from_f32<OutT>(sum);
                }
              }
            }
            if (rloc == 0) p.cnt[tile] = 0;
          }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.f;
        seg_units = 0;
      }
    }
  }
  if (*s_abort && tid == 0) atomicExch(p.status, 32);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(T5_TMEM_COLS));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn5() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

int sm_count5() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

constexpr int T5_SMEM_LIMIT = 227 * 1024;
// shared memory for an activation window of `asb` super-blocks
int smem_for(int asb) {
  return T5_WSTAGES * T5_WBYTES + asb * 2 * 2048 + 2 * asb * 8 * 64 + 1024;
}

// window each CTA needs: its own unit count (capped at a whole K)
bool plan(int64_t n, int64_t k, int* grid, int* asb) {
  const int nsb = (int)(k / 256);
  const int64_t ntiles = (n + T5_ROWS - 1) / T5_ROWS;
  const int64_t units = ntiles * nsb;
  int g = sm_count5();
  if (units < g) g = (int)units;
  const int64_t per = (units + g - 1) / g;
  const int64_t per_min = units / g;
  if (per_min < 1 || (nsb + per_min - 1) / per_min + 1 > 4) return false;   // the partial buffer holds 4 contributors per tile
  const int need = (int)(per >= nsb ? nsb : per);
  if (smem_for(need) > T5_SMEM_LIMIT) return false;
  *grid = g;
  *asb = need;
  return true;
}

template <int NT, typename OutT>
int launch5(const Tc5Params& p, const CUtensorMap& wmap, const CUtensorMap& qmap, int grid, int smem, cudaStream_t st) {
  auto kern = gemv_tc5_q4k_kernel<NT, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T5_SMEM_LIMIT));
    attr_set = true;
  }
  kern<<<grid, T5_THREADS, smem, st>>>(p, wmap, qmap);
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

}  // namespace

bool gemv_tc5_supported(const void* W, int type, int64_t n, int64_t k) {
  if (type != KQ_TYPE_Q4_K || (k % 256) || ((uintptr_t)W % 16)) return false;
  int g, asb;
  return encode_fn5() != nullptr && plan(n, k, &g, &asb);
}

// one pass of up to 16 tokens starting at m0 (m0 a multiple of 16)
int launch_gemv_tc5(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m_total, int64_t m0, int mcount,
                    void* y, int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st) {
  (void)type;
  EncodeTiledFn enc = encode_fn5();
  int grid, asb;
  if (!enc || !plan(n, k, &grid, &asb)) { set_error("tcgen05 GEMV: shape not covered"); return KQ_EUNSUPPORTED; }
  const int64_t rowbytes = k / 256 * 144;
  CUtensorMap wmap, qmap;
  {
    const cuuint64_t gdim[2] = {(cuuint64_t)(rowbytes / 4), (cuuint64_t)n};
    const cuuint64_t gstr[1] = {(cuuint64_t)rowbytes};
    const cuuint32_t box[2] = {36, T5_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(W), gdim, gstr, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("tcgen05 GEMV: weight tensor map failed (%d)", (int)r); return KQ_ECUDA; }
  }
  {
    const cuuint64_t gdim[2] = {(cuuint64_t)P.kpad, (cuuint64_t)m_total};
    const cuuint64_t gstr[1] = {(cuuint64_t)P.kpad};
    const cuuint32_t box[2] = {128, T5_NTOK};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&qmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)P.qs, gdim, gstr, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("tcgen05 GEMV: activation tensor map failed (%d)", (int)r); return KQ_ECUDA; }
  }
  Tc5Params p;
  p.n = (int)n; p.nsb = (int)(k / 256); p.ntiles = (int)((n + T5_ROWS - 1) / T5_ROWS);
  p.units = (int64_t)p.ntiles * p.nsb; p.m0 = (int)m0; p.mcount = mcount; p.asb_cap = asb;
  p.dT = P.dT; p.zT = mmq ? P.zs8 : P.z32; p.nb32tot = (int)(P.kpad / 32);
  p.y = y; p.stride_y = stride_y; p.part = P.part; p.cnt = P.cnt; p.status = P.status;
  const int smem = smem_for(asb);
#define KQ_T5(NT_)                                                                      \
  switch (y_dtype) {                                                                    \
    case KQ_F32: return launch5<NT_, float>(p, wmap, qmap, grid, smem, st);             \
    case KQ_F16: return launch5<NT_, __half>(p, wmap, qmap, grid, smem, st);            \
    case KQ_BF16: return launch5<NT_, __nv_bfloat16>(p, wmap, qmap, grid, smem, st);    \
  }
  if (mcount <= 4) { KQ_T5(4) } else if (mcount <= 8) { KQ_T5(8) } else { KQ_T5(16) }
#undef KQ_T5
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace kq
