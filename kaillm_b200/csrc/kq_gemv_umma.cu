// Decode GEMV on the 5th-generation tensor cores: the integer dots of 128 weight rows x 16 tokens x 32 weights are
// formed by tcgen05.mma.kind::i8 with the accumulators in tensor memory, so the CUDA cores only unpack the wire bytes
// and apply the per-block scales.
//
//   y[tok, row] = sum over 32-blocks b of  d8[tok, b] * (d[row] * sc[row, b] * I[tok, row, b])  -  min terms
//   I[tok, row, b] = sum_{i<32} q[row, 32 b + i] * a[tok, 32 b + i]      (exact, int32, in TMEM)
//
// with the fp32 combine of the reference's vec_dot functions (vllm_gguf_plugin/csrc/gguf/vecdotq.cuh:328-379 for Q4_K):
// sumf_d += d8 * (I * sc), sumf_m += d8 * (S * m), result d * sumf_d - dmin * sumf_m per super-block.
//
// Work is cut into units of (128 rows, one super-block of 256 weights); the units of all row tiles, in row-tile-major
// order, are split evenly over the CTAs (one per SM), so a row tile may be shared by a few CTAs.  Those write fp32
// partial sums in slots numbered by position; the CTA that arrives last adds the slots in that order (the result does
// not depend on timing) and stores the outputs.
//
//   warp 12      producer: per unit the bytes of the tile's 128 rows as 16-byte asynchronous copies (cp.async; a tiled
//                TMA box of 128 x 144 bytes took ~840 cycles to issue, one bulk copy per row 4.6 us per unit) plus the
//                unit's slice of the activation tables - codes in the tensor core's K-major core-matrix order, d8 and the min-term
//                sums token-minor - into a ring of shared-memory stages
//   warps 0-3    unpack: thread = weight row; nibbles -> int8 codes -> tensor memory (tcgen05.st) as the A operand;
//                while the tensor core works, the same thread adds up the row's min terms of the unit
//   warps 13-14  one lane each issues 4 of the unit's 8 MMAs (128 x 16 x 32, A from tensor memory, B = the staged codes
//                through a shared-memory descriptor), each into its own 16 accumulator columns; tcgen05.commit
//                signals "this unit's MMAs complete": accumulators ready and A slot free
//   warps 4-11   combine: thread = (weight row, half of the unit's 8 blocks): reads the integer dots back
//                (tcgen05.ld), scales them and keeps 16 fp32 sums; at the end of a row tile the two halves meet in
//                shared memory and lanes = consecutive rows store the outputs
//
// Every wait is bounded; a wait that gives up sets a status word, all roles leave their loops, tensor memory is
// released and the CTA returns.
#ifdef UM_TRACE
#include <cstdio>
#endif
#include "kq_common.cuh"
#include "kq_tma.cuh"

namespace kq {

namespace {

#include "kq_tile_common.cuh"

// wait with the cycles spent in it added to a counter when built with -DUM_TRACE (diagnostic builds only)
template <int SL>
__device__ __forceinline__ bool um_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, long long& waited) {
#ifdef UM_TRACE
  const long long t0 = clock64();
  const bool r = bar_wait<SL>(bar, parity, abort_flag);
  waited += clock64() - t0;
  return r;
#else
  return bar_wait<SL>(bar, parity, abort_flag);
#endif
}

constexpr int UM_ROWS = 128;                 // weight rows per tile = UMMA M = TMEM lanes
constexpr int UM_TOK = 16;                   // tokens per pass = UMMA N
constexpr int UM_UNPACK_WARPS = 4, UM_COMBINE_WARPS = 8;
constexpr int UM_WARP_PRODUCER = 12, UM_PRODUCER_WARPS = 2;   // warps 12-13 fetch, 14-15 issue the MMAs (half of a unit's blocks each)
constexpr int UM_WARP_MMA = 14, UM_MMA_WARPS = 2;
constexpr int UM_THREADS = 16 * 32;
constexpr int UM_NA = 2, UM_ND = 3;          // A slots (64 columns each) and accumulator buffers (128 columns each) in TMEM
constexpr int UM_NDONE = 6;                  // "MMAs of unit q complete" barriers: a multiple of both ring depths
constexpr uint32_t UM_TMEM_COLS = 512, UM_TMEM_A = 0, UM_TMEM_D = 128;
constexpr int UM_HEADER = 1024;
constexpr int UM_XCH_BYTES = 4 * UM_ROWS * 17 * 4;        // two sets of two buffers: the upper half's and the unpack warps' sums
                                                          // on their way to the lower half's threads
constexpr int UM_ACT_BYTES = 4096 + 3 * 512;              // per unit: codes 4 KB, d8, d8 * code sums, raw sums (512 B each)
constexpr int UM_MAX_STAGES = 8;
constexpr int UM_SMEM_LIMIT = 232448;
constexpr int UM_PART_SLOTS = KQ_PART_SLOTS;

template <int QT> struct UmUnit;
template <> struct UmUnit<KQ_TYPE_Q4_K> { static constexpr int BYTES = 144, SROW = 144; };

struct UmmaParams {
  const uint8_t* W;
  int64_t rowbytes;
  int n, nunit, ntiles;          // rows, super-blocks per row, row tiles
  int total, upc;                // units in all, units per CTA
  const uint8_t* qsu;            // this pass's unit tables [k/256][KQ_UNIT_TABLE]
  int zoff;                      // where the min-term sums start in a staged table: d8 * code sum, or the raw fp16 sum (MMQ flavour)
  int m0, mcount, stages, prefetch;
  int use_box;                   // 1: the unit's weight bytes arrive by one tiled TMA copy (rows 16-byte aligned), 0: by cp.async
  void* y;
  int64_t stride_y;
  float* part;
  int* cnt;
  int* status;
};

// Two fp32 values in one 64-bit register (the packed fp32 instructions of sm_100 take and return such pairs; keeping
// the accumulators packed avoids moving halves around)
using f2 = unsigned long long;
__device__ __forceinline__ f2 pk(float lo, float hi) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f2 pki(int lo, int hi) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ float2 unpk(f2 v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
__device__ __forceinline__ f2 fma2p(f2 a, f2 b, f2 c) {
  f2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f2 add2p(f2 a, f2 b) {
  f2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// (float)v0, (float)v1 for |v| < 2^22: integer add onto the magic exponent, then one packed subtraction
__device__ __forceinline__ f2 int2_to_f2(int v0, int v1, f2 neg_magic) {
  return add2p(pki(v0 + (int)TL_MAGIC_I, v1 + (int)TL_MAGIC_I), neg_magic);
}
__device__ __forceinline__ ulonglong2 lds128p(uint32_t a) { return *reinterpret_cast<const ulonglong2*>(tl_smem + a); }

__device__ __forceinline__ void um_tmem_st32(uint32_t taddr, const uint32_t (&a)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]),
        "r"(a[9]), "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(a[16]), "r"(a[17]), "r"(a[18]),
        "r"(a[19]), "r"(a[20]), "r"(a[21]), "r"(a[22]), "r"(a[23]), "r"(a[24]), "r"(a[25]), "r"(a[26]), "r"(a[27]), "r"(a[28]),
        "r"(a[29]), "r"(a[30]), "r"(a[31]) : "memory");
}
__device__ __forceinline__ void um_tmem_ld32(uint32_t taddr, int (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void um_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// How a row tile's outputs leave the CTAs that share it: tile t's units are [t * U, (t + 1) * U); CTA c holds units
// [c * upc, (c + 1) * upc).  first/last = the CTAs holding the tile's first/last unit.
__device__ __forceinline__ void tile_share(int t, int U, int upc, int& first, int& last) {
  first = (t * U) / upc;
  last = ((t + 1) * U - 1) / upc;
}

// NV = ceil(tokens / 4): the combine arithmetic covers 4 NV tokens (the MMAs always cover 16)
template <int QT, int NV, typename OutT>
__global__ void __launch_bounds__(UM_THREADS, 1) gemv_umma_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap wmap) {
  using UU = UmUnit<QT>;
  uint8_t* const smem = tl_smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + UM_HEADER - 32);
  volatile int* s_last = reinterpret_cast<volatile int*>(smem + UM_HEADER - 16);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + UM_HEADER - 8);
  float* sX = reinterpret_cast<float*>(smem + UM_HEADER);   // [2 flush parities][2 writers][128 rows][17]
  uint8_t* ring = smem + UM_HEADER + UM_XCH_BYTES;
  constexpr int RAW_BYTES = UM_ROWS * UU::SROW;
  constexpr int STAGE_BYTES = RAW_BYTES + UM_ACT_BYTES;
  constexpr int XBUF = UM_ROWS * 17;   // floats per exchange buffer

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  const int u0 = blockIdx.x * p.upc;
  const int u1 = min(u0 + p.upc, p.total);
  const int U = p.nunit;
  const int nq = u1 - u0;
  // barriers: full[S], empty[S], afull[NA], done[NDONE], dempty[ND], xa[2], xb[2], xc, xd
  const uint32_t bar_full = s_u32(bars), bar_empty = s_u32(bars + UM_MAX_STAGES), bar_afull = s_u32(bars + 2 * UM_MAX_STAGES),
                 bar_done = bar_afull + 8 * UM_NA, bar_dempty = bar_done + 8 * UM_NDONE,
                 bar_xa = bar_dempty + 8 * UM_ND, bar_xb = bar_xa + 16, bar_xc = bar_xb + 16, bar_xd = bar_xc + 8;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { bar_init(bar_full + 8 * s, p.use_box ? 1 : 32 * UM_PRODUCER_WARPS + 1); bar_init(bar_empty + 8 * s, UM_COMBINE_WARPS + UM_UNPACK_WARPS); }
    for (int a = 0; a < UM_NA; ++a) bar_init(bar_afull + 8 * a, UM_UNPACK_WARPS);
    for (int i = 0; i < UM_NDONE; ++i) bar_init(bar_done + 8 * i, UM_MMA_WARPS);
    for (int d = 0; d < UM_ND; ++d) bar_init(bar_dempty + 8 * d, UM_COMBINE_WARPS);
    for (int f = 0; f < 2; ++f) {
      bar_init(bar_xa + 8 * f, UM_COMBINE_WARPS / 2 + UM_UNPACK_WARPS);   // the upper half's and the unpack warps' sums are in shared memory
      bar_init(bar_xb + 8 * f, UM_COMBINE_WARPS / 2);                     // the lower half has read them
    }
    bar_init(bar_xc, UM_COMBINE_WARPS / 2);   // the lower half's partial sums are in global memory
    bar_init(bar_xd, 1);                      // the CTA has been counted in at the row tile's counter
    *s_abort = 0;
    *s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "r"(UM_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tbase = *tmem_slot;
  pdl_trigger();
  long long tw[4] = {0, 0, 0, 0};   // cycles spent waiting, per barrier kind (reported by diagnostic builds only)
#ifdef UM_TRACE
  const long long t_begin = clock64();
#endif

  if (warp >= UM_WARP_PRODUCER && warp < UM_WARP_PRODUCER + UM_PRODUCER_WARPS) {
    const int pw = warp - UM_WARP_PRODUCER;
    // ------------------------------------------------------------------ producer
    // The unit's bytes of the tile's 128 rows as 16-byte asynchronous copies: chunk c = (row c / CPR, piece c % CPR) goes
    // to c * 16 of the stage, so a warp-wide copy reads the segments of three to four consecutive rows.  Each lane's
    // copies signal the stage's barrier when they land.  The weights do not depend on the launch before this one: the
    // first stages are requested before pdl_wait(), the activation tables (one lane, bulk copies) after it.
    constexpr int CPR = UU::SROW / 16;               // chunks per row
    constexpr int NCH = UM_ROWS * CPR / (32 * UM_PRODUCER_WARPS);   // chunks per lane
    static_assert(UM_ROWS * CPR % (32 * UM_PRODUCER_WARPS) == 0, "chunks divide over the lanes");
    uint32_t off[NCH];   // byte offset of this lane's chunks from the tile's first row
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = (i * UM_PRODUCER_WARPS + pw) * 32 + lane, row = c / CPR;
      off[i] = (uint32_t)row * (uint32_t)p.rowbytes + (uint32_t)(c - row * CPR) * 16u;
    }
    auto issue_rows = [&](int q) {
      const int u = u0 + q, tile = u / U, j = u - tile * U, slot = q % S;
      if (p.use_box) {
        // one tiled copy: box = 128 rows x the unit's bytes of each row, rows land SROW bytes apart; rows past n arrive
        // as zeros and count all the same
        if (pw == 0 && lane == 0) {
          bar_expect_tx(bar_full + 8 * slot, (uint32_t)STAGE_BYTES);
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
              ::"r"(s_u32(ring + (size_t)slot * STAGE_BYTES)), "l"(&wmap), "r"(j * UU::BYTES), "r"(tile * UM_ROWS),
                "r"(bar_full + 8 * slot) : "memory");
        }
        return;
      }
      const int rows = min(UM_ROWS, p.n - tile * UM_ROWS);
      const uint32_t lim = (uint32_t)rows * (uint32_t)p.rowbytes;   // rows past n re-read the tile's last row (never used)
      const uint8_t* src = p.W + (size_t)tile * UM_ROWS * p.rowbytes + (size_t)j * UU::BYTES;
      const uint32_t dst = s_u32(ring + (size_t)slot * STAGE_BYTES) + (uint32_t)(pw * 32 + lane) * 16u;
      if (rows == UM_ROWS) {
#pragma unroll
        for (int i = 0; i < NCH; ++i)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 512 * UM_PRODUCER_WARPS), "l"(src + off[i]) : "memory");
      } else {   // the tensor's last tile
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const uint32_t o = off[i] < lim ? off[i] : off[i] - (off[i] / (uint32_t)p.rowbytes - (uint32_t)(rows - 1)) * (uint32_t)p.rowbytes;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 512 * UM_PRODUCER_WARPS), "l"(src + o) : "memory");
        }
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_full + 8 * slot) : "memory");
    };
    auto issue_tables = [&](int q) {
      if (lane != 0 || pw != 0) return;
      const int u = u0 + q, tile = u / U, j = u - tile * U, slot = q % S;
      const uint32_t dst = s_u32(ring + (size_t)slot * STAGE_BYTES + RAW_BYTES);
      if (!p.use_box) bar_expect_tx(bar_full + 8 * slot, (uint32_t)UM_ACT_BYTES);
      copy_g2s(dst, p.qsu + (size_t)j * KQ_UNIT_TABLE, UM_ACT_BYTES, bar_full + 8 * slot);
    };
    const int pre = min(min(p.prefetch, S), nq);
    for (int q = 0; q < pre; ++q) issue_rows(q);
    pdl_wait();
    for (int q = 0; q < pre; ++q) issue_tables(q);
    for (int q = pre; q < nq; ++q) {
      if (q >= S && !um_wait<32>(bar_empty + 8 * (q % S), (uint32_t)(((q / S) - 1) & 1), s_abort, tw[0])) { if (lane == 0) atomicExch(p.status, 31); break; }
      issue_rows(q);
      issue_tables(q);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this warp is in flight when the CTA leaves
  } else if (warp >= UM_WARP_MMA) {
    // ------------------------------------------------------------------ MMA issuers (blocks 4 w .. 4 w + 3 of every unit)
    if (lane == 0) {
      const int w = warp - UM_WARP_MMA;
      // D = s32, A = B = s8, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(UM_TOK >> 3) << 17) | ((uint32_t)(UM_ROWS >> 4) << 24);
      // the unit's codes: [16 chunks of 16 weights][16 tokens][16 bytes]; a core matrix (8 tokens x 16 bytes) is
      // 128 contiguous bytes, the next 8 tokens follow at +128 (SBO), the next 16 weights at +256 (LBO); no swizzle
      const uint64_t desc_hi = ((uint64_t)(256 >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | (1ull << 46);
      for (int q = 0; q < nq; ++q) {
        const int slot = q % S, a = q % UM_NA, d = q % UM_ND;
        // (the stage's bytes are complete: the unpack warps waited for them before they raised afull)
        bool ok = um_wait<32>(bar_afull + 8 * a, (uint32_t)((q / UM_NA) & 1), s_abort, tw[1]) &&
                  (q < UM_ND || um_wait<32>(bar_dempty + 8 * d, (uint32_t)(((q / UM_ND) - 1) & 1), s_abort, tw[2]));
        if (!ok) { atomicExch(p.status, 32); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t baddr = s_u32(ring + (size_t)slot * STAGE_BYTES + RAW_BYTES);
#pragma unroll
        for (int bb = 0; bb < 8 / UM_MMA_WARPS; ++bb) {
          const int b = w * (8 / UM_MMA_WARPS) + bb;
          const uint64_t bdesc = (uint64_t)(((baddr + b * 512) & 0x3FFFF) >> 4) | desc_hi;
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
              ::"r"(tbase + UM_TMEM_D + d * 128 + b * 16), "r"(tbase + UM_TMEM_A + a * 64 + b * 8), "l"(bdesc), "r"(idesc), "r"(0u)
              : "memory");
        }
        um_commit(bar_done + 8 * (q % UM_NDONE));   // accumulators ready (combine warps) and A slot free (unpack warps)
      }
    }
  } else if (warp < UM_UNPACK_WARPS) {
    // ------------------------------------------------------------------ unpack: wire bytes -> int8 codes in TMEM; min terms
    const int r = warp * 32 + lane;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    f2 accm[2 * NV];   // - dmin * sum over blocks of m * (min-term sum of the token), all units of the row tile so far
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) accm[i] = 0ull;
    int flush = 0;
    for (int q = 0; q < nq; ++q) {
      const int slot = q % S, a = q % UM_NA;
      const int u = u0 + q, j = u % U;
      if (!um_wait<32>(bar_full + 8 * slot, (uint32_t)((q / S) & 1), s_abort, tw[0]) ||
          (q >= UM_NA && !um_wait<32>(bar_done + 8 * ((q - UM_NA) % UM_NDONE), (uint32_t)(((q - UM_NA) / UM_NDONE) & 1), s_abort, tw[1]))) {
        if (lane == 0) atomicExch(p.status, 33);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t st = (uint32_t)(ring - smem) + (uint32_t)slot * STAGE_BYTES;
      const uint32_t raw = st + (uint32_t)r * UU::SROW;
      if constexpr (QT == KQ_TYPE_Q4_K) {
        // qs[32 j + i], i < 32: low nibbles = weights 64 j + i (block 2 j), high nibbles = weights 64 j + 32 + i
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t o[32];
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const uint4 w0 = lds128(raw + 16 + (hh * 2 + jj) * 32), w1 = lds128(raw + 32 + (hh * 2 + jj) * 32);
            const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              o[jj * 16 + i] = w[i] & 0x0F0F0F0Fu;
              o[jj * 16 + 8 + i] = (w[i] >> 4) & 0x0F0F0F0Fu;
            }
          }
          um_tmem_st32(tbase + lane_base + UM_TMEM_A + a * 64 + hh * 32, o);
        }
      }
      // the min terms of this unit, while the stores to tensor memory are on their way
      if constexpr (QT == KQ_TYPE_Q4_K) {
        {
          const uint4 hd = lds128(raw);
          const float dmin = __half2float(__ushort_as_half((unsigned short)(hd.x >> 16)));
          const uint32_t mlo = hd.z & 0x3F3F3F3Fu, mhi = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
          f2 um[2 * NV];
#pragma unroll
          for (int i = 0; i < 2 * NV; ++i) um[i] = 0ull;
          const uint32_t zta = st + RAW_BYTES + (uint32_t)p.zoff;
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const float mf = __uint_as_float(byte_of(b < 4 ? mlo : mhi, b & 3) | 0x4B000000u) - 8388608.0f;   // (float) of a byte
            const f2 m2 = pk(mf, mf);
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              const ulonglong2 z8 = lds128p(zta + b * 64 + v * 16);
              um[v * 2] = fma2p(m2, z8.x, um[v * 2]);
              um[v * 2 + 1] = fma2p(m2, z8.y, um[v * 2 + 1]);
            }
          }
          const f2 nd2 = pk(-dmin, -dmin);
#pragma unroll
          for (int i = 0; i < 2 * NV; ++i) accm[i] = fma2p(nd2, um[i], accm[i]);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(bar_afull + 8 * a);
      __syncwarp();
      if (lane == 0) bar_arrive(bar_empty + 8 * slot);
      if (j != U - 1 && q != nq - 1) continue;
      // ---- end of the CTA's share of this row tile: hand the min terms to the lower combine half
      const int fb = flush & 1;
      if (flush >= 2 && !um_wait<32>(bar_xb + 8 * fb, (uint32_t)(((flush >> 1) - 1) & 1), s_abort, tw[2])) break;
      float* dst = sX + (fb * 2 + 1) * XBUF + r * 17;
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) { const float2 t = unpk(accm[i]); dst[2 * i] = t.x; dst[2 * i + 1] = t.y; accm[i] = 0ull; }
      __syncwarp();
      if (lane == 0) bar_arrive(bar_xa + 8 * fb);
      ++flush;
    }
  } else {
    // ------------------------------------------------------------------ combine
    const int cw = warp - UM_UNPACK_WARPS;        // 0..7
    const int quad = cw & 3, h = cw >> 2;         // TMEM lane quadrant (= warp % 4), half of the unit's blocks
    const int r = quad * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    OutT* y = reinterpret_cast<OutT*>(p.y);
    f2 acc[2 * NV];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) acc[i] = 0ull;
    const f2 neg_magic = pk(-TL_MAGIC_F, -TL_MAGIC_F);
    uint32_t xph2 = 0;   // parity of the barriers used only by flushes of shared row tiles
    int flush = 0;
    bool ok = true;
    for (int q = 0; q < nq && ok; ++q) {
      const int slot = q % S, d = q % UM_ND;
      const int u = u0 + q, tile = u / U, j = u - tile * U;
      if (!um_wait<32>(bar_full + 8 * slot, (uint32_t)((q / S) & 1), s_abort, tw[0])) { if (lane == 0) atomicExch(p.status, 34); ok = false; break; }
      const uint32_t st = (uint32_t)(ring - smem) + (uint32_t)slot * STAGE_BYTES;
      const uint32_t dta = st + RAW_BYTES + 4096 + h * 4 * 64;
      // this row's scales for blocks 4 h .. 4 h + 3
      float dd = 0.f;
      uint32_t scw = 0;
      if constexpr (QT == KQ_TYPE_Q4_K) {
        const uint4 hd = lds128(st + (uint32_t)r * UU::SROW);
        dd = __half2float(__ushort_as_half((unsigned short)(hd.x & 0xFFFFu)));
        scw = h == 0 ? (hd.y & 0x3F3F3F3Fu) : ((hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u));
      }
      f2 ud[2 * NV];
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) ud[i] = 0ull;
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {
        // the activation scales of this pair of blocks (they do not depend on the MMAs: loaded before the wait)
        ulonglong2 d8[2][NV];
#pragma unroll
        for (int bb = 0; bb < 2; ++bb)
#pragma unroll
          for (int v = 0; v < NV; ++v) d8[bb][v] = lds128p(dta + (pr * 2 + bb) * 64 + v * 16);
        if (pr == 0) {
          if (!um_wait<32>(bar_done + 8 * (q % UM_NDONE), (uint32_t)((q / UM_NDONE) & 1), s_abort, tw[1])) { if (lane == 0) atomicExch(p.status, 35); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        int I[32];
        um_tmem_ld32(tbase + lane_base + UM_TMEM_D + d * 128 + (h * 4 + pr * 2) * 16, I);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (pr == 1) {
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) { bar_arrive(bar_dempty + 8 * d); bar_arrive(bar_empty + 8 * slot); }   // accumulators and stage read
        }
#pragma unroll
        for (int bb = 0; bb < 2; ++bb) {
          // float(I * sc) * d8: the integer multiply-add lands I * sc (< 2^22) on the magic exponent - conversion and
          // scaling in one instruction (measured: an integer add + a packed multiply by sc * d8 instead costs 9% more
          // instructions, the compiler turns the adds into multiply-adds on the same pipe)
          const int sc = (int)byte_of(scw, pr * 2 + bb);
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            ud[v * 2] = fma2p(int2_to_f2(I[bb * 16 + v * 4] * sc, I[bb * 16 + v * 4 + 1] * sc, neg_magic), d8[bb][v].x, ud[v * 2]);
            ud[v * 2 + 1] = fma2p(int2_to_f2(I[bb * 16 + v * 4 + 2] * sc, I[bb * 16 + v * 4 + 3] * sc, neg_magic), d8[bb][v].y, ud[v * 2 + 1]);
          }
        }
      }
      if (!ok) break;
      {
        const f2 dd2 = pk(dd, dd);
#pragma unroll
        for (int i = 0; i < 2 * NV; ++i) acc[i] = fma2p(dd2, ud[i], acc[i]);
      }
      if (j != U - 1 && q != nq - 1) continue;

      // ---- the CTA's share of this row tile is complete: the three partial sums of a row meet in shared memory
      // (exchange buffers and their barriers alternate between two sets, so the writers run one flush ahead)
      const int fb = flush & 1;
      const uint32_t fph = (uint32_t)((flush >> 1) & 1);
      if (h == 1) {
        if (flush >= 2 && !um_wait<32>(bar_xb + 8 * fb, fph ^ 1u, s_abort, tw[2])) { ok = false; break; }
        float* dst = sX + (fb * 2) * XBUF + r * 17;
#pragma unroll
        for (int i = 0; i < 2 * NV; ++i) { const float2 t = unpk(acc[i]); dst[2 * i] = t.x; dst[2 * i + 1] = t.y; }
        __syncwarp();
        if (lane == 0) bar_arrive(bar_xa + 8 * fb);
      } else {
        if (!um_wait<32>(bar_xa + 8 * fb, fph, s_abort, tw[2])) { if (lane == 0) atomicExch(p.status, 36); ok = false; break; }
        float v[4 * NV];
        const float* s0 = sX + (fb * 2) * XBUF + r * 17;
        const float* s1 = s0 + XBUF;
#pragma unroll
        for (int i = 0; i < 2 * NV; ++i) {
          const float2 t = unpk(acc[i]);
          v[2 * i] = (t.x + s0[2 * i]) + s1[2 * i];
          v[2 * i + 1] = (t.y + s0[2 * i + 1]) + s1[2 * i + 1];
        }
        __syncwarp();
        if (lane == 0) bar_arrive(bar_xb + 8 * fb);
        const int row = tile * UM_ROWS + r;
        int cf, cl;
        tile_share(tile, U, p.upc, cf, cl);
        const int ncontrib = cl - cf + 1;
        bool store = ncontrib == 1;
        if (ncontrib > 1) {
          // shared row tile: partial sums into this CTA's slot; the CTA that arrives last adds the slots in order
          const int myslot = (int)blockIdx.x - cf;
          if (row < p.n) {
#pragma unroll
            for (int t = 0; t < 4 * NV; ++t)
              if (t < p.mcount) __stcg(p.part + ((size_t)myslot * 16 + t) * p.n + row, v[t]);
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) bar_arrive(bar_xc);
          if (!um_wait<32>(bar_xc, xph2, s_abort, tw[3])) { if (lane == 0) atomicExch(p.status, 37); ok = false; break; }
          if (cw == 0 && lane == 0) {   // all four warps' partial sums are fenced: count the CTA in
            const int last = atomicAdd(p.cnt + tile, 1) == ncontrib - 1;
            if (last) p.cnt[tile] = 0;   // ready for the next launch on this scratch
            *s_last = last;
            bar_arrive(bar_xd);
          }
          if (!um_wait<32>(bar_xd, xph2, s_abort, tw[3])) { if (lane == 0) atomicExch(p.status, 38); ok = false; break; }
          store = *s_last != 0;
          xph2 ^= 1;
          if (store) {
            __threadfence();
            if (row < p.n) {
#pragma unroll
              for (int t = 0; t < 4 * NV; ++t) v[t] = 0.f;
              for (int c = 0; c < ncontrib; ++c) {   // slot order: the sum does not depend on who arrived when
                float pv[4 * NV];
#pragma unroll
                for (int t = 0; t < 4 * NV; ++t) pv[t] = t < p.mcount ? __ldcg(p.part + ((size_t)c * 16 + t) * p.n + row) : 0.f;
#pragma unroll
                for (int t = 0; t < 4 * NV; ++t) v[t] += pv[t];
              }
            }
          }
        }
        if (store && row < p.n) {
#pragma unroll
          for (int t = 0; t < 4 * NV; ++t)
            if (t < p.mcount) y[(size_t)(p.m0 + t) * p.stride_y + row] = from_f32<OutT>(v[t]);
        }
      }
      ++flush;
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) acc[i] = 0ull;
    }
  }

  // ---------------------------------------------------------------------- exit: every role comes here
#ifdef UM_TRACE
  if (blockIdx.x == 1 && lane == 0 && (warp == 0 || warp == 4 || warp == 8 || warp >= UM_WARP_PRODUCER))
    printf("warp %d units %d total %lld wait0 %lld wait1 %lld wait2 %lld wait3 %lld\n", warp, u1 - u0, clock64() - t_begin, tw[0], tw[1], tw[2], tw[3]);
#endif
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(UM_TMEM_COLS));
  }
}

}  // namespace

namespace {

struct UmmaConfig { int grid, upc, stages, smem, total, ntiles, nunit; };

bool make_umma_config(int type, int64_t n, int64_t k, UmmaConfig& c) {
  if (type != KQ_TYPE_Q4_K) return false;
  if (k % 256 || n <= 0 || n > (1 << 30)) return false;
  const int sms = sm_count();
  c.nunit = (int)(k / 256);
  c.ntiles = (int)((n + UM_ROWS - 1) / UM_ROWS);
  const int64_t total = (int64_t)c.ntiles * c.nunit;
  if (total > (1ll << 30) || c.ntiles > KQ_CNT_SLOTS) return false;
  c.total = (int)total;
  // a row tile may be shared by at most UM_PART_SLOTS CTAs: floor((U - 1) / upc) + 2 <= slots
  int upc = (c.total + sms - 1) / sms;
  // whole row tiles per CTA (no shared tiles, no partial sums) when that keeps at least 85% of the SMs' rounds busy
  {
    const int rounds = (c.ntiles + sms - 1) / sms;
    if ((int64_t)c.ntiles * 100 >= (int64_t)rounds * sms * 85) upc = rounds * c.nunit;
  }
  const int floor_upc = (c.nunit + UM_PART_SLOTS - 2) / (UM_PART_SLOTS - 1);
  if (upc < floor_upc) upc = floor_upc;
  c.upc = upc;
  c.grid = (c.total + upc - 1) / upc;
  const int stage = UM_ROWS * UmUnit<KQ_TYPE_Q4_K>::SROW + UM_ACT_BYTES;
  c.stages = (UM_SMEM_LIMIT - UM_HEADER - UM_XCH_BYTES) / stage;
  if (c.stages > UM_MAX_STAGES) c.stages = UM_MAX_STAGES;
  c.smem = UM_HEADER + UM_XCH_BYTES + c.stages * stage;
  return c.stages >= 3;
}

template <int QT, int NV, typename OutT>
int launch_umma(const UmmaParams& p, const UmmaConfig& c, cudaStream_t st) {
  auto kern = gemv_umma_kernel<QT, NV, OutT>;
  CUtensorMap map;
  memset(&map, 0, sizeof(map));
  if (p.use_box) {
    // the weight tensor as [n rows][row bytes] of uint8; a box is one unit of 128 rows
    EncodeTiledFn enc = encode_fn();
    if (!enc) { set_error("tensor-memory GEMV: cuTensorMapEncodeTiled is not available"); return KQ_ECUDA; }
    const cuuint64_t gdim[2] = {(cuuint64_t)p.rowbytes, (cuuint64_t)p.n};
    const cuuint64_t gstr[1] = {(cuuint64_t)p.rowbytes};
    const cuuint32_t box[2] = {(cuuint32_t)UmUnit<QT>::BYTES, (cuuint32_t)UM_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(p.W), gdim, gstr, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("tensor-memory GEMV: cuTensorMapEncodeTiled failed (%d)", (int)r); return KQ_ECUDA; }
  }
  static DeviceOnce configured;
  if (configured.first_time()) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_SMEM_LIMIT));
    configured.done();
  }
  KQ_CUDA_TRY(launch_pdl(kern, dim3(c.grid), dim3(UM_THREADS), (size_t)c.smem, st, options().pdl != 0, p, map));
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT>
int launch_umma_typed(const UmmaParams& p, const UmmaConfig& c, int y_dtype, cudaStream_t st) {
  const int nv = (p.mcount + 3) / 4;
#define KQ_UM_NV(T) (nv <= 1 ? launch_umma<QT, 1, T>(p, c, st) : (nv == 2 ? launch_umma<QT, 2, T>(p, c, st) : launch_umma<QT, 4, T>(p, c, st)))
  switch (y_dtype) {
    case KQ_F32: return KQ_UM_NV(float);
    case KQ_F16: return KQ_UM_NV(__half);
    case KQ_BF16: return KQ_UM_NV(__nv_bfloat16);
  }
#undef KQ_UM_NV
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace

bool gemv_umma_supported(const void* W, int type, int64_t n, int64_t k) {
  if ((uintptr_t)W % 16) return false;
  UmmaConfig c;
  return make_umma_config(type, n, k, c);
}

// one pass of up to 16 tokens starting at m0 (a multiple of 16)
int launch_gemv_umma(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m0, int mcount, void* y,
                     int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st) {
  UmmaConfig c;
  if (!make_umma_config(type, n, k, c)) { set_error("tensor-memory GEMV: shape or format not covered"); return KQ_EUNSUPPORTED; }
  if (!P.qsu) { set_error("tensor-memory GEMV: the activations were prepared without its tables (set the option first)"); return KQ_EINVAL; }
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  UmmaParams p;
  p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.n = (int)n; p.nunit = c.nunit; p.ntiles = c.ntiles;
  p.total = c.total; p.upc = c.upc;
  const int64_t pass = m0 >> 4;
  p.qsu = (const uint8_t*)P.qsu + (size_t)pass * (size_t)(P.kpad / 256) * KQ_UNIT_TABLE;
  p.zoff = mmq ? 4096 + 1024 : 4096 + 512;
  p.m0 = (int)m0; p.mcount = mcount; p.stages = c.stages;
  p.prefetch = options().pdl < c.stages ? options().pdl : c.stages;
  p.y = y; p.stride_y = stride_y; p.part = P.part; p.cnt = P.cnt; p.status = P.status;
  p.use_box = options().umma_box && (p.rowbytes % 16) == 0 && UmUnit<KQ_TYPE_Q4_K>::BYTES % 16 == 0;
  return launch_umma_typed<KQ_TYPE_Q4_K>(p, c, y_dtype, st);
}

}  // namespace kq
