// Prefill GEMM (M >= ~32 tokens): dequantize-on-the-fly + tcgen05 (5th-gen tensor core) MMA with TMEM accumulators.
//
//   y[tok, row] = sum_k  w^[row, k] * x^[tok, k]   (+ sum_b c[row, b] * s8[tok, b])
//   w^ = the weight dequantized to fp16 with the op order of ggml_dequantize
//        (vllm_gguf_plugin/csrc/gguf/dequantize.cuh:156-196 etc.), x^ = fp16(d8 * q8) of the q8_1-quantized
//        activation (gguf_kernel.cu:32-69).  fp16 operands, fp32 accumulation in TMEM: rel-L2 ~3e-4 to the
//        integer-dot arithmetic of the reference's MMQ kernels (bf16 operands would give 2e-3).
//   The reference forms Q4_0's "-8" offset and MMQ-flavoured Q4_K's min term from the fp16 sum of the RAW
//   activations of each 32-block (s8), not from the quantized codes (vecdotq.cuh:46-66, 353-379); a dense
//   product cannot express that, and the difference (1e-2 for Q4_0, 1e-3 for Q4_K) would break the 1e-3 gate.
//   For those cases w^ is formed without the offset/min and extra K steps multiply the per-block coefficient
//   c[row, b] (-8*d, or -dmin*m) with s8[tok, b] into the same accumulator.
//
//   CTA tile  2 x 128 weight rows (two accumulators, UMMA M = 128: one TMEM lane per row) x BN = 128 tokens (UMMA N),
//             both accumulators fed by the same activation tile; K step = 128
//   warps 0-15 thread = (weight row of one of the two row tiles, one of the step's two 64-weight atoms): dequantizes 64
//             weights to packed fp16 registers and writes them to TMEM with tcgen05.st - the A operand never touches
//             shared memory.  Q4_K and Q6_K wire bytes reach the threads through a shared-memory stage filled with
//             coalesced cp.async pieces (one super-block column of the CTA's 256 rows per stage); the other formats are
//             read straight from global/L2, prefetched one step ahead.  After the K loop the same threads read the
//             accumulators back (tcgen05.ld) and store y (lanes = consecutive rows: coalesced).
//   warp 16   one lane fetches the x^ tile [BN x 128] of each K step with two TMA tiled loads (128-byte swizzle)
//   warp 17   one lane issues the MMAs: per K step 8 x tcgen05.mma.kind::f16 (128 x 128 x 16) per row tile, A from TMEM,
//             B through a shared-memory descriptor; tcgen05.commit signals "buffers free" and, at the end,
//             "accumulators complete".
//   TMEM: 256 accumulator columns (2 x 128) + an A ring of 2 slots x 128 columns; shared memory: a B ring of 5 steps x
//   32 KB.  Every mbarrier wait is bounded; on give-up a status word is set, TMEM is released and the CTA returns.
#include "kq_common.cuh"
#include "kq_tma.cuh"

namespace kq {
namespace {

constexpr int BM = 128;         // UMMA M: weight rows per accumulator (one TMEM lane per row)
constexpr int KSTEP = 128;      // k per pipeline step (two swizzle atoms)
constexpr int ATOM = 64;        // k per 128-byte swizzle atom (fp16)
constexpr int DQ_WARPS = 16;    // dequantizing warps
constexpr int GEMM_THREADS = (DQ_WARPS + 2) * 32;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TMEM_D = 0;                 // accumulators: 256 columns
constexpr uint32_t TMEM_A = 256;               // A ring: 256 columns
constexpr int W6_ROW = 232;                    // Q6_K: bytes per staged row (216-byte aligned window of a 210-byte block, padded)

// Two tile shapes, same TMEM budget (256 accumulator columns + 256 columns of A ring):
//   narrow  2 row tiles x 128 tokens: warp w unpacks for row tile w>>3, atom (w>>2)&1 of EVERY step; an unpacked
//           weight meets 128 tokens.  For m <= 128.
//   wide    1 row tile x 256 tokens (UMMA N = 256): the two groups of 8 warps take alternate K steps (group w>>3
//           serves the steps of its parity), so an unpacked weight meets 256 tokens - half the unpacking
//           instructions per flop, twice the activation bytes per flop (64 KB per step through a ring of 3).
template <bool WIDE>
struct Tile {
  static constexpr int RT = WIDE ? 1 : 2;          // accumulators (row tiles) per CTA
  static constexpr int BN = WIDE ? 256 : 128;      // tokens per CTA = UMMA N
  static constexpr int NA = WIDE ? 4 : 2;          // A ring slots
  static constexpr int NB = WIDE ? 3 : 5;          // B ring stages
  static constexpr int SLOT = RT * 64;             // TMEM columns per A slot: row tile t, atom a at t * 64 + a * 32
  static constexpr int B_STAGE = BN * KSTEP * 2;   // 32 / 64 KB
  static constexpr int A_ARRIVALS = WIDE ? DQ_WARPS / 2 : DQ_WARPS;
  static constexpr int W4_STAGE = RT * BM * 144;   // Q4_K: one super-block column of the CTA's rows
  static constexpr int W6_STAGE = RT * BM * W6_ROW;
};
constexpr long long GEMM_WAIT_LIMIT = 1ll << 28;

__device__ const uint16_t c_iq3s_codes_g[512] = {
#include "kq_iq3s_codes.inc"
};

struct GemmParams {
  const uint8_t* W;
  int64_t rowbytes;
  int n, k, m;
  int ntok_tiles;
  int ncorr;          // extra K steps over the 32-block raw-sum table (0 = none)
  int nb32;           // k / 32
  void* y;
  int64_t stride_y;
  int* status;
  int half_fma;
  int stage6;         // Q6_K: rows and W are 8-byte aligned, the block columns go through shared memory
  const __half* ctab;  // Q4_0: dense table [n][ctab_stride] of -8 * d per 32-block (null: read the scales from W)
  int64_t ctab_stride;
  int stagew;         // Q8_0, Q4_0, Q2_K in the 128 x 256 tile: W is 16-byte aligned and k a multiple of 256, the columns go through shared memory
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
    if (clock64() - t0 > GEMM_WAIT_LIMIT) { *abort_flag = 1; return false; }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// ------------------------------------------------------------------------------------------------ dequantization
// 64 consecutive weights (k = 64*atom .. +63 of the 256-weight block or of 8 consecutive 32-weight blocks at `blk`)
// -> 32 packed fp16 pairs, with the fp16 operation order of ggml_dequantize.
__device__ __forceinline__ __half mul_sub_h(__half a, __half b, __half c, int fma) {
  return fma ? __hfma(a, b, __hneg(c)) : __hsub_rn(__hmul_rn(a, b), c);
}

// coefficient of the raw block sum for 32-block b of this row: Q4_0 -8*d, Q4_K -dmin*m (both fp16)
template <int QT>
__device__ __forceinline__ __half corr_coef(const uint8_t* __restrict__ wrow, int b) {
  if constexpr (QT == KQ_TYPE_Q4_0) {
    return __hmul_rn(__float2half_rn(-8.0f), __ushort_as_half(*reinterpret_cast<const uint16_t*>(wrow + (size_t)b * 18)));
  } else if constexpr (QT == KQ_TYPE_Q4_K) {
    const uint8_t* blk = wrow + (size_t)(b >> 3) * 144;
    const int j = b & 7;
    const uint8_t* q = blk + 4;
    const int mn = j < 4 ? (q[j + 4] & 63) : ((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    const __half dmin = __ushort_as_half(*reinterpret_cast<const uint16_t*>(blk + 2));
    return __hneg(__hmul_rn(dmin, __int2half_rn(mn)));
  } else {
    return __float2half_rn(0.f);
  }
}

template <int QT>
__device__ __noinline__ void corr_atom_scattered(const uint8_t* __restrict__ wrow, int atom, int nb32, uint32_t* out) {
  for (int i = 0; i < 32; ++i) {
    const int b = atom * 64 + 2 * i;
    const __half c0 = b < nb32 ? corr_coef<QT>(wrow, b) : __float2half_rn(0.f);
    const __half c1 = b + 1 < nb32 ? corr_coef<QT>(wrow, b + 1) : __float2half_rn(0.f);
    out[i] = h2_bits(__halves2half2(c0, c1));
  }
}

template <int QT>
__device__ __forceinline__ void corr_atom(const uint8_t* __restrict__ wrow, int atom, int nb32, const __half* __restrict__ crow,
                                          uint32_t (&out)[32]) {
  if (QT == KQ_TYPE_Q4_0 && crow != nullptr) {
    // the row's coefficients were laid out densely (zero past the last block) by q4_0_coef_kernel: 128 contiguous bytes
    const uint4* c = reinterpret_cast<const uint4*>(crow + (size_t)atom * 64);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 v = __ldg(c + i);
      out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
    return;
  }
  if constexpr (QT == KQ_TYPE_Q4_K) {
    // 64 coefficients = 8 super-blocks x 8 sub-block mins; one 16-byte header load per super-block
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
      const int b0 = atom * 64 + sb * 8;
      uint4 h = make_uint4(0u, 0u, 0u, 0u);
      if (b0 < nb32) h = __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)(b0 >> 3) * 144));
      const __half ndmin = __hneg(__high2half(bits_h2(h.x)));
      const uint32_t mn[2] = {h.z & 0x3F3F3F3Fu, ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m0 = (int)((mn[j >> 1] >> (16 * (j & 1))) & 0xFFu), m1 = (int)((mn[j >> 1] >> (16 * (j & 1) + 8)) & 0xFFu);
        out[4 * sb + j] = h2_bits(__halves2half2(__hmul_rn(ndmin, __int2half_rn(m0)), __hmul_rn(ndmin, __int2half_rn(m1))));
      }
    }
  } else {
    // rare path (Q4_0 without its coefficient table): kept out of line so that its 64 scattered loads do not weigh on
    // the register allocation of the K loop
    uint32_t tmp[32];
    corr_atom_scattered<QT>(wrow, atom, nb32, tmp);
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = tmp[i];
  }
}

// CORR: leave the offset (Q4_0) / min (Q4_K) out of w^; it is applied through corr_atom steps instead
template <int QT, bool CORR>
__device__ __forceinline__ void dequant_atom(const uint8_t* __restrict__ blk, int atom, const uint32_t* grid, int fma,
                                             const uint4 (&pre)[3], uint32_t (&out)[32]) {
  if constexpr (QT == KQ_TYPE_Q4_K) {
    // atom a = sub-blocks 2a (low nibbles of qs[32a..32a+31]) and 2a+1 (high nibbles); 16-byte aligned block.
    // `pre` holds the block header and the atom's 32 nibble bytes, fetched one step ahead by the caller.
    const uint4 hdr = pre[0];
    const __half2 dm = bits_h2(hdr.x);
    const uint32_t scw = atom < 2 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u));
    const uint32_t mnw = atom < 2 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u));
    const int sh = 16 * (atom & 1);
    const __half d1 = __hmul_rn(__low2half(dm), __int2half_rn((int)((scw >> sh) & 0xFFu)));
    const __half d2 = __hmul_rn(__low2half(dm), __int2half_rn((int)((scw >> (sh + 8)) & 0xFFu)));
    const __half m1 = __hmul_rn(__high2half(dm), __int2half_rn((int)((mnw >> sh) & 0xFFu)));
    const __half m2 = __hmul_rn(__high2half(dm), __int2half_rn((int)((mnw >> (sh + 8)) & 0xFFu)));
    const __half2 d1v = __half2half2(d1), d2v = __half2half2(d2);
    const __half2 nm1 = __half2half2(__hneg(m1)), nm2 = __half2half2(__hneg(m2));
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const uint4 w0 = pre[1];
    const uint4 w1 = pre[2];
    const uint32_t wq[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t lo = wq[i] & 0x0F0F0F0Fu, hi = (wq[i] >> 4) & 0x0F0F0F0Fu;
      // bytes (n0, n1) -> half2 (1024+n0, 1024+n1), minus 1024: exact small integers in fp16
      const __half2 l01 = __hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x4140)), k1024);
      const __half2 l23 = __hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x4342)), k1024);
      const __half2 h01 = __hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x4140)), k1024);
      const __half2 h23 = __hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x4342)), k1024);
      if constexpr (CORR) {
        out[2 * i] = h2_bits(__hmul2_rn(d1v, l01));
        out[2 * i + 1] = h2_bits(__hmul2_rn(d1v, l23));
        out[16 + 2 * i] = h2_bits(__hmul2_rn(d2v, h01));
        out[16 + 2 * i + 1] = h2_bits(__hmul2_rn(d2v, h23));
      } else if (fma) {
        out[2 * i] = h2_bits(__hfma2(d1v, l01, nm1));
        out[2 * i + 1] = h2_bits(__hfma2(d1v, l23, nm1));
        out[16 + 2 * i] = h2_bits(__hfma2(d2v, h01, nm2));
        out[16 + 2 * i + 1] = h2_bits(__hfma2(d2v, h23, nm2));
      } else {
        out[2 * i] = h2_bits(__hadd2_rn(__hmul2_rn(d1v, l01), nm1));
        out[2 * i + 1] = h2_bits(__hadd2_rn(__hmul2_rn(d1v, l23), nm1));
        out[16 + 2 * i] = h2_bits(__hadd2_rn(__hmul2_rn(d2v, h01), nm2));
        out[16 + 2 * i + 1] = h2_bits(__hadd2_rn(__hmul2_rn(d2v, h23), nm2));
      }
    }
  } else {
    // general formats: decode two 32-weight sub-blocks to integer codes, then apply the fp16 op sequence per weight
    using F = Fmt<QT>;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int sb = 2 * atom + e;   // sub-block index relative to `blk` (for 32-weight blocks: block index)
      SubBlock s;
      decode_subblock<QT>(blk, sb, grid, s);
      // scale fields again, as fp16
      __half d = __float2half_rn(0.f), dmin = d;
      int sc[2] = {0, 0}, mn[2] = {0, 0};
      float fsc = 0.f;
      if constexpr (QT == KQ_TYPE_Q4_0) { d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(blk + (size_t)sb * 18)); }
      if constexpr (QT == KQ_TYPE_Q8_0) { d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(blk + (size_t)sb * 34)); }
      if constexpr (QT == KQ_TYPE_Q2_K) {
        d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(blk + 80));
        dmin = __ushort_as_half(*reinterpret_cast<const uint16_t*>(blk + 82));
        for (int h = 0; h < 2; ++h) { const int v = blk[2 * sb + h]; sc[h] = v & 15; mn[h] = v >> 4; }
      }
      if constexpr (QT == KQ_TYPE_Q6_K) {
        d = __ushort_as_half(*reinterpret_cast<const uint16_t*>(blk + 208));
        const int ip = sb >> 2, q4 = sb & 3;
        for (int h = 0; h < 2; ++h) sc[h] = (int8_t)blk[192 + 8 * ip + 2 * q4 + h];
      }
      if constexpr (QT == KQ_TYPE_IQ3_S) {
        const float dh = ld_h(blk);
        const uint32_t s4 = (blk[106 + (sb >> 1)] >> (4 * (sb & 1))) & 15u;
        fsc = __fmul_rn(__fmul_rn(dh, 0.5f + (float)s4), 0.5f);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        __half r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int h = (F::GROUP == 16) ? (i >> 2) : 0;
          const int code = (QT == KQ_TYPE_Q4_0 || QT == KQ_TYPE_Q2_K) ? (int)((s.v[i] >> (8 * j)) & 0xFFu)
                                                                      : (int)(int8_t)(s.v[i] >> (8 * j));
          if constexpr (QT == KQ_TYPE_Q4_0) r[j] = __hmul_rn(__int2half_rn(code), d);   // offset applied via corr steps
          if constexpr (QT == KQ_TYPE_Q8_0) r[j] = __hmul_rn(__int2half_rn(code), d);
          if constexpr (QT == KQ_TYPE_Q2_K) {
            const __half xq = __int2half_rn(sc[h] * code);
            const __half mp = __hmul_rn(dmin, __int2half_rn(mn[h]));
            r[j] = fma == 2 ? __hfma(__hneg(dmin), __int2half_rn(mn[h]), __hmul_rn(d, xq)) : mul_sub_h(d, xq, mp, fma);
          }
          if constexpr (QT == KQ_TYPE_Q6_K) r[j] = __hmul_rn(d, __int2half_rn(sc[h] * code));
          if constexpr (QT == KQ_TYPE_IQ3_S) r[j] = __float2half_rn(__fmul_rn(fsc, (float)code));
        }
        out[16 * e + 2 * i] = h2_bits(__halves2half2(r[0], r[1]));
        out[16 * e + 2 * i + 1] = h2_bits(__halves2half2(r[2], r[3]));
      }
    }
  }
}

// Q6_K atom from registers: ql = the 64 low-nibble bytes of the atom's half super-block (16 words), qh = its 32
// high-bit bytes (8 words), scw = its four int8 scales, p = which nibble / which pair of 2-bit fields (atom & 1).
// Same fp16 operation order as ggml_dequantize: half(sc * q) in one rounding, then * d.
__device__ __forceinline__ void dequant_q6k_regs(const uint32_t (&ql)[16], const uint32_t (&qh)[8], uint32_t scw, __half d,
                                                 int p, uint32_t (&out)[32]) {
  const __half2 k1056 = __half2half2(__ushort_as_half(0x6420));   // 1024 + 32
  const __half2 d2 = __half2half2(d);
  __half2 sc2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) sc2[i] = __half2half2(__int2half_rn((int)(int8_t)(scw >> (8 * i))));
#pragma unroll
  for (int run = 0; run < 2; ++run) {        // q4 = 2p + run: weights 32*run .. 32*run+31 of the atom
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t qlw = ql[8 * run + w] >> (4 * p);
      const uint32_t qhw = qh[w];
      const int sh = 4 * p + 2 * run;            // the 2-bit field of this run, moved to bits 4-5
      const uint32_t hi = sh <= 4 ? qhw << (4 - sh) : qhw >> (sh - 4);
      const uint32_t code = (qlw & 0x0F0F0F0Fu) | (hi & 0x30303030u);
      const __half2 q01 = __hsub2(bits_h2(__byte_perm(code, 0x64646464u, 0x4140)), k1056);
      const __half2 q23 = __hsub2(bits_h2(__byte_perm(code, 0x64646464u, 0x4342)), k1056);
      const __half2 s2 = sc2[2 * run + (w >> 2)];
      out[16 * run + 2 * w] = h2_bits(__hmul2_rn(d2, __hmul2_rn(q01, s2)));
      out[16 * run + 2 * w + 1] = h2_bits(__hmul2_rn(d2, __hmul2_rn(q23, s2)));
    }
  }
}

// Window staging of the 32-weight-block formats and Q2_K (128 x 256 tile only): per 256-weight column a row owns COLB wire
// bytes; the 16-byte aligned window around them goes to shared memory in 16-byte pieces, each unpacking thread pulls the
// words of its own 64-weight atom into registers and unpacks from there, two weights per fp16x2 instruction.
template <int QT> struct Win { static constexpr bool ON = false; enum { COLB = 16, PIECES = 1, SROW = 16, NG = 1 }; };
template <> struct Win<KQ_TYPE_Q8_0> { static constexpr bool ON = true; static constexpr int COLB = 272, PIECES = 17, SROW = 272, NG = 17; };
template <> struct Win<KQ_TYPE_Q4_0> { static constexpr bool ON = true; static constexpr int COLB = 144, PIECES = 9, SROW = 144, NG = 9; };
// Q2_K blocks are 4-byte aligned (84 = 4 * 21): a block starts 0, 4, 8 or 12 bytes into its window of 6 pieces
template <> struct Win<KQ_TYPE_Q2_K> { static constexpr bool ON = true; static constexpr int COLB = 84, PIECES = 6, SROW = 112, NG = 10; };

// bytes (b0, b1) and (b2, b3) of `w`, each plus 1024, as fp16 pairs (the bytes land in the mantissas of 0x6400)
__device__ __forceinline__ __half2 bytes01_plus1024(uint32_t w) { return bits_h2(__byte_perm(w, 0x64646464u, 0x4140)); }
__device__ __forceinline__ __half2 bytes23_plus1024(uint32_t w) { return bits_h2(__byte_perm(w, 0x64646464u, 0x4342)); }

// Q8_0 atom = two blocks = 68 bytes = 17 words g: block 0 {d at bytes 0-1, codes at 2-33}, block 1 {d at 34-35, codes at
// 36-67 = words 9..16}.  Signed codes: c ^ 0x80 = c + 128 as an unsigned byte, so 1024 + byte - 1152 = c exactly.
__device__ __forceinline__ void dequant_q8_0_regs(const uint32_t (&g)[17], uint32_t (&out)[32]) {
  const __half2 k1152 = __half2half2(__ushort_as_half(0x6480));
  const __half2 d0 = __half2half2(__low2half(bits_h2(g[0]))), d1 = __half2half2(__high2half(bits_h2(g[8])));
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t c0 = __byte_perm(g[j], g[j + 1], 0x5432) ^ 0x80808080u, c1 = g[9 + j] ^ 0x80808080u;
    out[2 * j] = h2_bits(__hmul2_rn(__hsub2(bytes01_plus1024(c0), k1152), d0));
    out[2 * j + 1] = h2_bits(__hmul2_rn(__hsub2(bytes23_plus1024(c0), k1152), d0));
    out[16 + 2 * j] = h2_bits(__hmul2_rn(__hsub2(bytes01_plus1024(c1), k1152), d1));
    out[16 + 2 * j + 1] = h2_bits(__hmul2_rn(__hsub2(bytes23_plus1024(c1), k1152), d1));
  }
}

// Q4_0 atom = two blocks = 36 bytes = 9 words: block 0 {d, qs at bytes 2-17}, block 1 {d at 18-19, qs at 20-35 = words
// 5..8}; weight j = low nibble of qs[j], weight j + 16 = high nibble.  d * q without the -8 (applied by the correction steps).
__device__ __forceinline__ void dequant_q4_0_regs(const uint32_t (&g)[9], uint32_t (&out)[32]) {
  const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const __half2 d = __half2half2(e ? __high2half(bits_h2(g[4])) : __low2half(bits_h2(g[0])));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t w = e ? g[5 + j] : __byte_perm(g[j], g[j + 1], 0x5432);
      const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
      out[16 * e + 2 * j] = h2_bits(__hmul2_rn(__hsub2(bytes01_plus1024(lo), k1024), d));
      out[16 * e + 2 * j + 1] = h2_bits(__hmul2_rn(__hsub2(bytes23_plus1024(lo), k1024), d));
      out[16 * e + 8 + 2 * j] = h2_bits(__hmul2_rn(__hsub2(bytes01_plus1024(hi), k1024), d));
      out[16 * e + 8 + 2 * j + 1] = h2_bits(__hmul2_rn(__hsub2(bytes23_plus1024(hi), k1024), d));
    }
  }
}

// Q2_K atom a4 of a super-block: half h = a4 >> 1 (qs bytes 32h..32h+31 = g[1..8]), 2-bit fields 2 * (a4 & 1) and
// 2 * (a4 & 1) + 1; g[0] = its four scale bytes (sc | mn << 4, one per 16 weights), g[9] = {d, dmin}.
// Same fp16 operations as the scalar path: half(sc * q) exact, then d * that minus dmin * mn in the order `fma` selects.
__device__ __forceinline__ void dequant_q2_k_regs(const uint32_t (&g)[10], int odd, int fma, uint32_t (&out)[32]) {
  const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
  const __half2 dm = bits_h2(g[9]);
  const __half2 d2 = __half2half2(__low2half(dm)), dmin2 = __half2half2(__high2half(dm));
#pragma unroll
  for (int run = 0; run < 2; ++run) {              // field 2 * odd + run: weights 32 * run .. + 31 of the atom
    const int sh = 2 * (2 * odd + run);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {               // 16 weights under one scale byte
      const uint32_t sb = (g[0] >> (8 * (2 * run + hh))) & 0xFFu;
      const __half2 sc2 = __half2half2(__int2half_rn((int)(sb & 15u))), mn2 = __half2half2(__int2half_rn((int)(sb >> 4)));
      const __half2 mp2 = __hmul2_rn(dmin2, mn2);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t code = (g[1 + 4 * hh + w] >> sh) & 0x03030303u;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const __half2 xq = __hmul2_rn(__hsub2(q ? bytes23_plus1024(code) : bytes01_plus1024(code), k1024), sc2);
          __half2 r;
          if (fma == 2) r = __hfma2(__hneg2(dmin2), mn2, __hmul2_rn(d2, xq));
          else if (fma) r = __hfma2(d2, xq, __hneg2(mp2));
          else r = __hsub2(__hmul2_rn(d2, xq), mp2);
          out[16 * run + 8 * hh + 2 * w + q] = h2_bits(r);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ kernel
template <int QT, bool CORR, typename OutT, bool WIDE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap smap) {
  using F = Fmt<QT>;
  using T = Tile<WIDE>;
  constexpr int RT = T::RT, BN = T::BN, NA = T::NA, NB = T::NB, A_SLOT_COLS = T::SLOT, B_STAGE_BYTES = T::B_STAGE;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sB = smem;                                            // NB stages; each atom [BN rows x 128 B] swizzled
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NB * B_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 27);
  uint32_t* s_grid = reinterpret_cast<uint32_t*>(bars + 32);     // IQ3_S codebook (2 KB)
  uint8_t* sW = smem + NB * B_STAGE_BYTES + (QT == KQ_TYPE_IQ3_S ? 4096 : 1024);                // staged super-block column of the CTA's rows (Q4_K 144 B, Q6_K 232 B per row)
  const uint32_t bar_bfull = smem_u32(bars), bar_bempty = smem_u32(bars + 8), bar_afull = smem_u32(bars + 16),
                 bar_aempty = smem_u32(bars + 20), bar_dfull = smem_u32(bars + 24);
  static_assert(NB <= 8 && NA <= 4, "barrier layout");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_tile = blockIdx.x / p.ntok_tiles, tok_tile = blockIdx.x % p.ntok_tiles;
  const int nmain = p.k / KSTEP;
  const int nsteps = nmain + (CORR ? p.ncorr : 0);

  if (tid == 0) {
    for (int i = 0; i < NB; ++i) { mbar_init(bar_bfull + 8 * i, 1); mbar_init(bar_bempty + 8 * i, 1); }
    for (int i = 0; i < NA; ++i) { mbar_init(bar_afull + 8 * i, T::A_ARRIVALS); mbar_init(bar_aempty + 8 * i, 1); }
    mbar_init(bar_dfull, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = tid; i < 512; i += GEMM_THREADS) s_grid[i] = iq3s_expand(c_iq3s_codes_g[i], KQ_IQ3S_TOP);
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tbase = *tmem_slot;

  if (warp == DQ_WARPS) {
    // -------------------------------------------------------------------------- activation loader (TMA)
    if (lane == 0) {
      for (int s = 0; s < nsteps; ++s) {
        const int buf = s % NB, fill = s / NB;
        if (fill > 0 && !mbar_wait(bar_bempty + 8 * buf, (uint32_t)((fill - 1) & 1), s_abort)) break;
        mbar_expect_tx(bar_bfull + 8 * buf, B_STAGE_BYTES);
#pragma unroll
        for (int a = 0; a < KSTEP / ATOM; ++a) {
          const uint32_t dst = smem_u32(sB + buf * B_STAGE_BYTES + a * (BN * 128));
          if (s < nmain) tma_load_2d(dst, &xmap, s * KSTEP + a * ATOM, tok_tile * BN, bar_bfull + 8 * buf);
          else tma_load_2d(dst, &smap, (s - nmain) * KSTEP + a * ATOM, tok_tile * BN, bar_bfull + 8 * buf);
        }
      }
    }
  } else if (warp == DQ_WARPS + 1) {
    // -------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = f32, A = B = f16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      for (int s = 0; s < nsteps && ok; ++s) {
        const int ab = s % NA, bb = s % NB;
        ok = mbar_wait(bar_bfull + 8 * bb, (uint32_t)((s / NB) & 1), s_abort) &&
             mbar_wait(bar_afull + 8 * ab, (uint32_t)((s / NA) & 1), s_abort);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int a = 0; a < KSTEP / ATOM; ++a) {
          // shared-memory descriptor: addr >> 4, LBO (unused with swizzle), SBO = 1024 B, version 1, 128-byte swizzle
          const uint32_t baddr = smem_u32(sB + bb * B_STAGE_BYTES + a * (BN * 128));
          const uint64_t bdesc = (uint64_t)((baddr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) |
                                 (1ull << 46) | (2ull << 61);
#pragma unroll
          for (int kk = 0; kk < ATOM / 16; ++kk) {
            const uint32_t accum = (s > 0 || a > 0 || kk > 0) ? 1u : 0u;
#pragma unroll
            for (int t = 0; t < RT; ++t) {   // every row tile against the same B tile
              const uint32_t ta = tbase + TMEM_A + ab * A_SLOT_COLS + t * 64 + a * 32 + kk * 8;
              asm volatile(
                  "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                  "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                  ::"r"(tbase + TMEM_D + t * BN), "r"(ta), "l"(bdesc + (uint64_t)((kk * 32) >> 4)), "r"(idesc), "r"(accum) : "memory");
            }
          }
        }
        // completion of everything issued so far frees this step's A slot and B stage
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_aempty + 8 * ab) : "memory");
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_bempty + 8 * bb) : "memory");
      }
      if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_dfull) : "memory");
    }
  } else {
    // -------------------------------------------------------------------------- dequantizers
    const int rloc = (warp & 3) * 32 + lane;          // row inside a row tile = TMEM lane
    const int half = (warp >> 2) & 1;                 // which of the step's two atoms
    const int grp = warp >> 3;                        // narrow: which of the CTA's row tiles; wide: which step parity
    const int t = WIDE ? 0 : grp;                     // row tile of this thread
    int row = (row_tile * RT + t) * BM + rloc;
    const bool row_ok = row < p.n;
    if (!row_ok) row = p.n - 1;                       // clamp: loads stay in bounds, the store is skipped
    const uint8_t* wrow = p.W + (size_t)row * p.rowbytes;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    constexpr int ATOMS_PER_BLK = F::BLK >= 256 ? 4 : 1;   // 32-weight formats: dequant_atom indexes blocks itself
    bool ok = true;
    const uint4 pre[3] = {};
    // Q4_K: the wire bytes of a super-block column of the CTA's rows (256 rows x 144 B) are staged through shared
    // memory by all dequantizing threads with 16-byte asynchronous copies (consecutive threads take consecutive
    // 16-byte pieces of a row, so the global reads coalesce), then every thread pulls its row's header and the two
    // 32-byte nibble runs of its two atoms into registers and the buffer is free for the next column while the two
    // K steps are unpacked.  The named barrier is reached by every dequantizing thread on every iteration, also
    // after a wait has given up (`ok` only guards the work), so it cannot be left waiting.
    constexpr int NE = WIDE ? 1 : 2;                  // atoms of a super-block column this thread unpacks
    uint4 hdr4 = {}, qa[NE][2] = {};
    uint32_t q6l[NE][16] = {}, q6h[NE][8] = {}, q6s[NE] = {};   // Q6_K: the thread's atoms of the current column
    __half q6d = __float2half_rn(0.f);
    const bool st6 = QT == KQ_TYPE_Q6_K && p.stage6 != 0;
    using WN = Win<QT>;
    constexpr bool WINQ = WIDE && WN::ON;              // a window-staged format in the tile shape that has room for it
    const bool stw = WINQ && p.stagew != 0;
    constexpr int DQ_THREADS = DQ_WARPS * 32;
    // pieces per row and column: Q4_K 9 x 16 B (the block), Q6_K 27 x 8 B (the 8-byte aligned window around the block),
    // window formats: 16-byte pieces of the 16-byte aligned window
    constexpr int PIECES = QT == KQ_TYPE_Q6_K ? 27 : WINQ ? WN::PIECES : 9;
    constexpr int PIECE_B = QT == KQ_TYPE_Q6_K ? 8 : 16;
    constexpr int SROW = QT == KQ_TYPE_Q6_K ? W6_ROW : WINQ ? WN::SROW : 144;
    constexpr int NCHUNK = (QT == KQ_TYPE_Q4_K || QT == KQ_TYPE_Q6_K || WINQ) ? (RT * BM * PIECES + DQ_THREADS - 1) / DQ_THREADS : 1;
    const int dq_tid = warp * 32 + lane;
    const uint8_t* csrc[NCHUNK];
    uint32_t cdst[NCHUNK];
    if (QT == KQ_TYPE_Q4_K || st6 || stw) {
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int c = dq_tid + i * DQ_THREADS;
        const int r = c / PIECES, part = c - PIECES * r;
        int grow = row_tile * RT * BM + r;
        if (grow >= p.n) grow = p.n - 1;
        // window formats: the row's start (the window is aligned per column when the copies are issued); the piece
        // index rides in the top byte of cdst
        csrc[i] = c < RT * BM * PIECES ? p.W + (size_t)grow * p.rowbytes + (WINQ ? 0 : part * PIECE_B) : nullptr;
        cdst[i] = smem_u32(sW + r * SROW + part * PIECE_B) | (WINQ ? (uint32_t)part << 24 : 0u);
      }
    }
    const bool holds_last_row = (row_tile + 1) * RT * BM >= p.n;   // rows past n are clamped to row n - 1
    const int last_sblk = p.k / 256 - 1;
    auto stage_block = [&](int sblk) {                          // issue the copies of super-block column sblk
      if constexpr (WINQ) {
        // The window of the LAST column of the LAST row may reach a few bytes past the tensor (Q2_K: up to 12).  Only a
        // CTA that holds that row, and only there, takes the careful path, where a piece reads just the bytes that
        // exist (the rest of its 16 bytes is zero-filled).
        const size_t col = (size_t)sblk * WN::COLB;
        const bool careful = holds_last_row && sblk == last_sblk;
        const uint8_t* wend = p.W + (size_t)p.n * p.rowbytes;
#pragma unroll
        for (int i = 0; i < NCHUNK; ++i)
          if (csrc[i]) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>((uintptr_t)(csrc[i] + col) & ~(uintptr_t)15) + ((cdst[i] >> 24) << 4);
            const uint32_t have = (!careful || src + 16 <= wend) ? 16u : (src < wend ? (uint32_t)(wend - src) : 0u);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(cdst[i] & 0xFFFFFFu), "l"(src), "r"(have) : "memory");
          }
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
      if constexpr (QT == KQ_TYPE_Q4_K) {
#pragma unroll
        for (int i = 0; i < NCHUNK; ++i)
          if (csrc[i]) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(cdst[i]), "l"(csrc[i] + (size_t)sblk * 144) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
      if constexpr (QT == KQ_TYPE_Q6_K) {
        const size_t col = ((size_t)sblk * 210) & ~(size_t)7;   // rows and W are 8-byte aligned: the same for every row
        // The aligned window of the LAST block of the LAST row may reach up to 6 bytes past the tensor.  Only a CTA
        // that holds that row, and only at that block, takes the careful path, where a piece reads just the bytes
        // that exist (the rest of its 8 bytes is zero-filled); everywhere else the plain 8-byte copies run.
        if (holds_last_row && sblk == last_sblk) {
          const uint8_t* wend = p.W + (size_t)p.n * p.rowbytes;
#pragma unroll
          for (int i = 0; i < NCHUNK; ++i)
            if (csrc[i]) {
              const uint8_t* src = csrc[i] + col;
              const uint32_t have = src + 8 <= wend ? 8u : (src < wend ? (uint32_t)(wend - src) : 0u);
              asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(cdst[i]), "l"(src), "r"(have) : "memory");
            }
        } else {
#pragma unroll
          for (int i = 0; i < NCHUNK; ++i)
            if (csrc[i]) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(cdst[i]), "l"(csrc[i] + col) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    };
    auto dq_barrier = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS) : "memory"); };
    uint32_t gq[WN::NG] = {};                         // window formats: the words of the thread's atom
    if (QT == KQ_TYPE_Q4_K || st6 || stw) stage_block(0);
    // narrow: one iteration per step.  wide: one iteration per PAIR of steps (= super-block column); the thread
    // unpacks for step 2 * it + grp only, but takes part in the staging of every column.
    const int niter = WIDE ? (nsteps + 1) / 2 : nsteps;
    for (int it = 0; it < niter; ++it) {
      const int s = WIDE ? 2 * it + grp : it;
      const int ab = s % NA, fill = s / NA;
      const bool new_col = WIDE ? (2 * it < nmain) : (s < nmain && (s & 1) == 0);
      const int col = WIDE ? it : (s >> 1);           // super-block column
      const int sel = WIDE ? 0 : (s & 1);             // which of the thread's pulled atoms this step uses
      // dequantize before waiting for the slot: the wire bytes do not depend on the pipeline state
      uint32_t v[32];
      if constexpr (QT == KQ_TYPE_Q4_K) {
        if (new_col) {
          asm volatile("cp.async.wait_group 0;" ::: "memory");
          dq_barrier();                               // the whole column has landed
          const uint8_t* mine = sW + (t * BM + rloc) * 144;
          hdr4 = *reinterpret_cast<const uint4*>(mine);
#pragma unroll
          for (int e = 0; e < NE; ++e) {              // narrow: atoms `half` (this step) and `half + 2` (next step); wide: atom 2 * grp + half
            const int a4 = WIDE ? 2 * grp + half : half + 2 * e;
            qa[e][0] = *reinterpret_cast<const uint4*>(mine + 16 + 32 * a4);
            qa[e][1] = *reinterpret_cast<const uint4*>(mine + 32 + 32 * a4);
          }
          dq_barrier();                               // everyone has its bytes: the buffer may be refilled
          if (2 * (col + 1) < nmain) stage_block(col + 1);
        }
      }
      if constexpr (QT == KQ_TYPE_Q6_K) {
        if (st6 && new_col) {
          asm volatile("cp.async.wait_group 0;" ::: "memory");
          dq_barrier();
          const uint32_t off = (uint32_t)(((size_t)col * 210) & 7);        // where the block starts inside its window
          const uint8_t* mine = sW + (t * BM + rloc) * W6_ROW + off;
          const uint32_t fsh = ((uint32_t)(uintptr_t)mine & 2u) << 3;      // 0 or 16: the same for all rows
          auto words = [&](const uint8_t* ptr, uint32_t* dst, int n) {     // n 32-bit words from a 2-byte aligned address
            const uint32_t* q = reinterpret_cast<const uint32_t*>((uintptr_t)ptr & ~(uintptr_t)3);
            uint32_t lo = q[0];
#pragma unroll
            for (int i = 0; i < n; ++i) { const uint32_t hi = q[i + 1]; dst[i] = __funnelshift_r(lo, hi, fsh); lo = hi; }
          };
#pragma unroll
          for (int e = 0; e < NE; ++e) {              // half super-block: narrow e (this step, next step), wide grp
            const int ip = WIDE ? grp : e;
            words(mine + 64 * ip, q6l[e], 16);
            words(mine + 128 + 32 * ip, q6h[e], 8);
            words(mine + 192 + 8 * ip + 4 * half, &q6s[e], 1);
          }
          q6d = *reinterpret_cast<const __half*>(mine + 208);
          dq_barrier();
          if (2 * (col + 1) < nmain) stage_block(col + 1);
        }
      }
      if constexpr (WINQ) {
        if (stw && new_col) {
          asm volatile("cp.async.wait_group 0;" ::: "memory");
          dq_barrier();
          const uint32_t off = (uint32_t)((uintptr_t)(wrow + (size_t)col * WN::COLB) & 15);   // where the column starts inside its window
          const uint8_t* mine = sW + rloc * WN::SROW + off;
          const int a4 = 2 * grp + half;
          if constexpr (QT == KQ_TYPE_Q2_K) {
            gq[0] = *reinterpret_cast<const uint32_t*>(mine + 4 * a4);
#pragma unroll
            for (int i = 0; i < 8; ++i) gq[1 + i] = *reinterpret_cast<const uint32_t*>(mine + 16 + 32 * grp + 4 * i);
            gq[9] = *reinterpret_cast<const uint32_t*>(mine + 80);
          } else {
#pragma unroll
            for (int i = 0; i < WN::NG; ++i) gq[i] = *reinterpret_cast<const uint32_t*>(mine + (WN::COLB / 4) * a4 + 4 * i);
          }
          dq_barrier();
          if (2 * (col + 1) < nmain) stage_block(col + 1);
        }
      }
      if (s >= nsteps) continue;                      // wide, odd number of steps: nothing left for this group
      if (s < nmain) {
        const int ga = s * (KSTEP / ATOM) + half;     // atom index along the row
        if constexpr (QT == KQ_TYPE_Q4_K) {
          const bool second = NE > 1 && sel;
          const uint4 cur[3] = {hdr4, second ? qa[NE - 1][0] : qa[0][0], second ? qa[NE - 1][1] : qa[0][1]};
          dequant_atom<QT, CORR>(nullptr, ga & 3, s_grid, p.half_fma, cur, v);
        } else if (st6) {
          if constexpr (QT == KQ_TYPE_Q6_K) {
            if (NE > 1 && sel) dequant_q6k_regs(q6l[NE - 1], q6h[NE - 1], q6s[NE - 1], q6d, half, v);
            else dequant_q6k_regs(q6l[0], q6h[0], q6s[0], q6d, half, v);
          }
        } else if (stw) {
          if constexpr (WINQ && QT == KQ_TYPE_Q8_0) dequant_q8_0_regs(gq, v);
          if constexpr (WINQ && QT == KQ_TYPE_Q4_0) dequant_q4_0_regs(gq, v);
          if constexpr (WINQ && QT == KQ_TYPE_Q2_K) dequant_q2_k_regs(gq, half, p.half_fma, v);
        } else {
          const uint8_t* blk = F::BLK >= 256 ? wrow + (size_t)(ga / ATOMS_PER_BLK) * F::BYTES
                                             : wrow + (size_t)ga * 2 * F::BYTES;
          dequant_atom<QT, CORR>(blk, F::BLK >= 256 ? (ga % ATOMS_PER_BLK) : 0, s_grid, p.half_fma, pre, v);
        }
      } else {
        corr_atom<QT>(wrow, (s - nmain) * (KSTEP / ATOM) + half, p.nb32, p.ctab ? p.ctab + (size_t)row * p.ctab_stride : nullptr, v);
      }
      if (ok && fill > 0) ok = mbar_wait(bar_aempty + 8 * ab, (uint32_t)((fill - 1) & 1), s_abort);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_st32(tbase + TMEM_A + lane_base + ab * A_SLOT_COLS + t * 64 + half * 32, v);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_afull + 8 * ab);
      }
    }
    // -------------------------------------------------------------------------- epilogue: warp w takes the 64
    // accumulator columns [64 * (w >> 2), +64) of its 32 lanes (narrow: that is its own row tile's accumulator)
    if (ok && mbar_wait(bar_dfull, 0, s_abort)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      OutT* y = reinterpret_cast<OutT*>(p.y);
      const int cbase = (warp >> 2) * 64;
#pragma unroll 1
      for (int c0 = cbase; c0 < cbase + 64; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tbase + TMEM_D + lane_base + c0, r);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int tok = tok_tile * BN + c0 - t * BN + j;
          if (row_ok && tok < p.m) y[(size_t)tok * p.stride_y + row] = from_f32<OutT>(__uint_as_float(r[j]));
        }
      }
    }
  }
  if (*s_abort && tid == 0) atomicExch(p.status, 16);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(TMEM_COLS));
}

// Q4_0: out[row][b] = -8 * d(row, b) as fp16 for b < nb, 0 up to `stride`.  One warp per row; consecutive lanes read
// consecutive blocks' scales (18 bytes apart: every sector of the row is touched once).
__global__ void __launch_bounds__(256) q4_0_coef_kernel(const uint8_t* __restrict__ W, int64_t rowbytes, int n, int nb,
                                                        __half* __restrict__ out, int64_t stride) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const uint8_t* wrow = W + (size_t)row * rowbytes;
  __half* o = out + (size_t)row * stride;
  for (int b = lane; b < (int)stride; b += 32)
    o[b] = b < nb ? __hmul_rn(__float2half_rn(-8.0f), __ushort_as_half(*reinterpret_cast<const uint16_t*>(wrow + (size_t)b * 18)))
                  : __float2half_rn(0.f);
}

// ------------------------------------------------------------------------------------------------ host

template <int QT, bool CORR, typename OutT, bool WIDE>
int launch(const GemmParams& p, const CUtensorMap& map, const CUtensorMap& smap, int grid, cudaStream_t st) {
  using T = Tile<WIDE>;
  auto kern = gemm_tc_kernel<QT, CORR, OutT, WIDE>;
  constexpr int WSTAGE = QT == KQ_TYPE_Q4_K ? T::W4_STAGE : QT == KQ_TYPE_Q6_K ? T::W6_STAGE : (WIDE && Win<QT>::ON) ? BM * Win<QT>::SROW : 0;
  constexpr int smem = T::NB * T::B_STAGE + (QT == KQ_TYPE_IQ3_S ? 4096 : 1024) + WSTAGE;   // barriers (+ IQ3_S codebook), then the weight stage
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static DeviceOnce attr_set;   // the attribute belongs to the (function, device) pair
  if (attr_set.first_time()) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set.done();
  }
  kern<<<grid, GEMM_THREADS, smem, st>>>(p, map, smap);
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT, bool CORR>
int launch_out(const GemmParams& p, const CUtensorMap& map, const CUtensorMap& smap, int grid, int y_dtype, bool wide, cudaStream_t st) {
  switch (y_dtype) {
    case KQ_F32: return wide ? launch<QT, CORR, float, true>(p, map, smap, grid, st) : launch<QT, CORR, float, false>(p, map, smap, grid, st);
    case KQ_F16: return wide ? launch<QT, CORR, __half, true>(p, map, smap, grid, st) : launch<QT, CORR, __half, false>(p, map, smap, grid, st);
    case KQ_BF16: return wide ? launch<QT, CORR, __nv_bfloat16, true>(p, map, smap, grid, st) : launch<QT, CORR, __nv_bfloat16, false>(p, map, smap, grid, st);
  }
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace

bool gemm_tc_staged(int type) {
  return type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q6_K || type == KQ_TYPE_Q8_0 || type == KQ_TYPE_Q4_0 || type == KQ_TYPE_Q2_K;
}

// The tensor-core GEMM needs whole 256-weight K steps and 16-byte aligned Q4_K blocks; everything else is general.
bool gemm_tc_supported(const void* W, int type, int64_t n, int64_t k) {
  if (!type_is_core(type)) return false;
  if (k % KSTEP) return false;
  if (type == KQ_TYPE_Q4_K && ((uintptr_t)W % 16)) return false;
  return encode_fn() != nullptr;
}

// xh: fp16 [m][kpad] dequantized activations (written by the quantizer)
int launch_gemm_tc(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m, void* y, int y_dtype,
                   int64_t stride_y, bool mmq, cudaStream_t st) {
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  EncodeTiledFn enc = encode_fn();
  if (!enc) { set_error("tensor-core GEMM: cuTensorMapEncodeTiled is not available"); return KQ_ECUDA; }
  CUtensorMap map;
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)m};
  const cuuint64_t gstr[1] = {(cuuint64_t)P.kpad * 2};
  // tile shape: option gemm_wide 0 = always 256 rows x 128 tokens; 2 = always 128 rows x 256 tokens; 1 = the latter when
  // more than 128 tokens come, and at every m for the staged formats (measured at 96 tokens: Q4_K 17408x5120 39.8
  // against 58.3 us, Q6_K 17408x5120 53.4 against 142 us - unpacking, not the tensor pipe, is what a step costs)
  const bool wide = options().gemm_wide == 2 || (options().gemm_wide == 1 && (m > 128 || gemm_tc_staged(type)));
  const int BN = wide ? Tile<true>::BN : Tile<false>::BN, RT = wide ? Tile<true>::RT : Tile<false>::RT;
  const cuuint32_t box[2] = {ATOM, (cuuint32_t)BN};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)P.xh, gdim, gstr, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("tensor-core GEMM: cuTensorMapEncodeTiled failed (%d)", (int)r); return KQ_ECUDA; }
  // raw block sums s8 as fp16 [m][kpad/32]; columns past k/32 read as zero (tensor-map bounds)
  CUtensorMap smap;
  const cuuint64_t sdim[2] = {(cuuint64_t)(k / 32), (cuuint64_t)m};
  const cuuint64_t sstr[1] = {(cuuint64_t)(P.kpad / 32) * 2};
  const CUresult r2 = enc(&smap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)P.s8h, sdim, sstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r2 != CUDA_SUCCESS) { set_error("tensor-core GEMM: cuTensorMapEncodeTiled failed (%d)", (int)r2); return KQ_ECUDA; }
  const bool corr = type == KQ_TYPE_Q4_0 || (type == KQ_TYPE_Q4_K && mmq);
  GemmParams p;
  p.ncorr = corr ? (int)((k / 32 + KSTEP - 1) / KSTEP) : 0;
  p.nb32 = (int)(k / 32);
  p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.n = (int)n; p.k = (int)k; p.m = (int)m;
  p.ntok_tiles = (int)((m + BN - 1) / BN);
  p.y = y; p.stride_y = stride_y; p.status = P.status; p.half_fma = options().half_fma;
  p.stage6 = type == KQ_TYPE_Q6_K && ((uintptr_t)W % 8) == 0 && (p.rowbytes % 8) == 0;
  p.stagew = ((uintptr_t)W % 16) == 0 && (k % 256) == 0;
  p.ctab = nullptr; p.ctab_stride = 0;
  if (type == KQ_TYPE_Q4_0 && P.w16 != nullptr) {
    q4_0_coef_kernel<<<(unsigned)((n + 7) / 8), 256, 0, st>>>((const uint8_t*)W, p.rowbytes, (int)n, p.nb32, P.w16, P.w16_stride);
    options().launches += 1;
    KQ_CUDA_TRY(cudaGetLastError());
    p.ctab = P.w16; p.ctab_stride = P.w16_stride;
  }
  const int grid = (int)((n + RT * BM - 1) / (RT * BM)) * p.ntok_tiles;
  switch (type) {
    case KQ_TYPE_Q4_0: return launch_out<KQ_TYPE_Q4_0, true>(p, map, smap, grid, y_dtype, wide, st);
    case KQ_TYPE_Q8_0: return launch_out<KQ_TYPE_Q8_0, false>(p, map, smap, grid, y_dtype, wide, st);
    case KQ_TYPE_Q2_K: return launch_out<KQ_TYPE_Q2_K, false>(p, map, smap, grid, y_dtype, wide, st);
    case KQ_TYPE_Q4_K: return corr ? launch_out<KQ_TYPE_Q4_K, true>(p, map, smap, grid, y_dtype, wide, st)
                                   : launch_out<KQ_TYPE_Q4_K, false>(p, map, smap, grid, y_dtype, wide, st);
    case KQ_TYPE_Q6_K: return launch_out<KQ_TYPE_Q6_K, false>(p, map, smap, grid, y_dtype, wide, st);
    case KQ_TYPE_IQ3_S: return launch_out<KQ_TYPE_IQ3_S, false>(p, map, smap, grid, y_dtype, wide, st);
  }
  return KQ_EUNSUPPORTED;
}

}  // namespace kq
