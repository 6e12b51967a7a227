// Decode GEMV for 3..16 tokens per pass (all six formats): int8 mma.sync, every warp of the CTA on every stage.
//
//   grid      one CTA per SM, in `ks` groups; group s works on K slice s of every weight row it owns (ks is the
//             smallest of 1, 2, 4 whose activation slice leaves room for a ring of >= 4 stages)
//   stage     8 consecutive weight rows x the CTA's K slice.  With ks == 1 that is one contiguous piece of the
//             wire tensor and ONE bulk copy; otherwise eight row segments of a few KB each
//   CTA       16 consumer warps + 1 reducer warp + 1 producer warp
//   consumer  the stage's super-blocks are dealt round-robin over the sixteen warps (unit = stage x super-block,
//             unit u belongs to warp u % 16, so the load evens out over a few stages).  Lane (g, t) unpacks the
//             weights of row g and reads the activations of token g (and g + 8 for 9..16 tokens); it ends up
//             with the outputs of row g for tokens 2t, 2t+1, so the block scales it needs are those of its own row.
//             Q4_K: the 16 A rows of an m16n8k32 mma are the 8 weight rows twice - low nibbles (sub-block 2i) in
//             rows 0-7, high nibbles (sub-block 2i+1) in rows 8-15 - so the unpacked words are the A fragment
//             as they stand; one mma against the activations of each of the two sub-blocks, half of each result
//             unused.  Q6_K: the two 16-weight scale groups of a 32-block sit in the two row halves of one mma.
//             The scales are applied in fp32 on the way into the warp's 8 x 16 partial tile.  The Q4_K min term
//             is a small GEMM over the eight sub-blocks of a super-block (mins 0..63, exact in tf32) x
//             (d8 * block sum, split hi + lo): two tf32 mmas per super-block and token half.
//   reducer   adds the sixteen partial tiles of a stage in warp order (deterministic) and stores the outputs.
//             With ks > 1 it stores fp32 partials instead; after its last stage it raises the tiles' counters
//             (one fence, one round of atomics), and the consumer warps, idle by then, finish in parallel the
//             tiles at which this CTA arrived last, adding the splits in split order.
//   rings     stage ring: full (copy bytes) / empty (16 consumer arrivals);  partial-tile ring of two buffers:
//             red_full (16 arrivals) / red_empty (reducer), so a consumer runs at most two stages ahead
//
// Every consumer visits every stage, so a parity wait is never more than one phase behind.  All waits are
// bounded (about 2^27 clocks) and sleep between polls: the waiter raises a CTA-wide abort flag and a status
// word, every warp leaves its loop and the producer waits, again bounded, for the copies it has in flight.
// No branch around an mma depends on the lane: the alignment cases of Q6_K are either the same for all 32
// lanes or handled without a branch.
//
// Combine: vllm_gguf_plugin/csrc/gguf/vecdotq.cuh:328-379 (Q4_K), 447-491 (Q6_K).
#include "kq_common.cuh"

namespace kq {

namespace {

constexpr int TL_ROWS = 8;
constexpr int TL_CW = 16;                         // consumer warps
constexpr int TL_THREADS = (TL_CW + 2) * 32;      // + reducer + producer
constexpr int TL_HEADER = 1024;
constexpr int TL_TILE_BYTES = 768;                // the reducer's transpose tile: 16 tokens x 12 floats
constexpr int TL_NRED = 2;                        // partial-tile buffers (a power of two)
constexpr int TL_SLEEP_C = 64, TL_SLEEP_R = 200, TL_SLEEP_P = 400;   // ns between polls: consumers, reducer, producer
constexpr int TL_MAX_STAGES = 16;
constexpr int TL_SMEM_LIMIT = 232448;

__device__ const uint16_t c_iq3s_codes_t[512] = {
#include "kq_iq3s_codes.inc"
};
constexpr int TL_GRID_BYTES = 2048;               // IQ3_S: the expanded 512-entry codebook in shared memory

struct TileParams {
  const uint8_t* W;
  int64_t rowbytes;
  int n, nblk, ks, ntiles;
  int stages, row_stride, stage_bytes, contig;
  int a_stride, a_bytes, d_bytes, z_bytes;
  const int8_t* qs;
  const float* dT;
  const float* zT;
  int zpb;            // z entries per 32-block in zT (2 for Q2_K: one per 16-weight group)
  int kpad, nb32tot;
  int m0, mcount, prefetch;
  void* y;
  int64_t stride_y;
  float* part;
  int* cnt;
  int* status;
  // fused all-gather (g_world > 1): the outputs go, as columns g_col0 .., straight into every rank's row-major [M, N]
  // buffer by plain peer stores; the last CTA to finish raises this call's flag on every rank and waits for theirs
  void* peer_y[8];
  uint32_t* peer_flags[8];
  uint32_t* g_epoch;
  uint32_t* g_done;
  int* g_status;   // set (and never cleared here) when the wait for a peer's flag ran out
  int g_ll;        // 1: no hand-shake - the outputs are their own arrival flags (the consumer polls against the sentinel)
  uint4* g_reset;  // g_ll: local buffer to refill with the sentinel (the one the previous producer consumed), or null
  uint32_t g_reset_n;   // ... in 16-byte units
  int g_slot, g_rank, g_world;
  int64_t g_col0;
};

struct TileConfig {
  int ks, grid, stages, row_stride, stage_bytes, contig, a_stride, a_bytes, d_bytes, z_bytes, smem;
};

#include "kq_tile_common.cuh"

struct TileView {       // byte offsets (into the dynamic shared memory) of the CTA's activation slice
  uint32_t sA;          // [tokens][a_stride] codes
  uint32_t a_stride;
  uint32_t sD;          // [32-block][16 tokens] fp32 d8
  uint32_t sZ;          // [32-block][16 tokens] fp32 min-term factor (Q4_K)
};

// Lane (g, t) of a consumer warp: B-operand column g = token g (and g + 8 in the second half), A-operand row g =
// weight row g of the stage; it ends up with the outputs of row g for tokens 2t, 2t+1 (and 8+2t, 8+2t+1).
//
// ---------------------------------------------------------------------------------------------- Q4_K unit
// One super-block (pg: its first byte in row g).  The 16 A rows of an m16n8k32 mma are the 8 weight rows twice:
// rows 0-7 carry the low nibbles of 32 bytes (sub-block 2il), rows 8-15 the high nibbles (sub-block 2il+1), so
// the unpacked words drop into the A fragment as they are.  One mma against the activations of sub-block 2il
// (its rows 8-15 are ignored) and one against those of 2il+1 (rows 0-7 ignored).  Inside a 32-block the k
// index is permuted (fragment k = 4t+i <-> position 8t+i, 16+4t+i <-> 8t+4+i) on both operands, so a lane
// reads its two activation registers with one 64-bit load.  b0: first 32-block of the super-block in the slice.
template <int NH>
__device__ __forceinline__ void unit_q4k(uint32_t pg, int b0, const TileView& A, int g, int t, float (&acc)[4]) {
  const uint4 h = lds128(pg);   // {d, dmin}, scales[12]
  const uint32_t sc[2] = {h.y & 0x3F3F3F3Fu, (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)};
  const uint32_t mn[2] = {h.z & 0x3F3F3F3Fu, ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)};
  float u[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t tok = A.sA + (uint32_t)g * A.a_stride + (uint32_t)b0 * 32u + 8u * (uint32_t)t;
  const uint32_t dsc = A.sD + ((uint32_t)b0 * 16u + 2u * (uint32_t)t) * 4u;
#pragma unroll
  for (int il = 0; il < 4; ++il) {
    const uint2 w = lds64(pg + 16 + 32 * il + 8 * t);
    const uint32_t a0 = w.x & 0x0F0F0F0Fu, a1 = (w.x >> 4) & 0x0F0F0F0Fu;
    const uint32_t a2 = w.y & 0x0F0F0F0Fu, a3 = (w.y >> 4) & 0x0F0F0F0Fu;
    const int sl = (int)byte_of(sc[il >> 1], (2 * il) & 3), sh = (int)byte_of(sc[il >> 1], (2 * il + 1) & 3);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      const uint2 xl = lds64(tok + hf * 8 * A.a_stride + (2 * il) * 32);
      const uint2 xh = lds64(tok + hf * 8 * A.a_stride + (2 * il + 1) * 32);
      int Dl[4], Dh[4];
      mma_i8_k32(Dl, a0, a1, a2, a3, xl.x, xl.y);
      mma_i8_k32(Dh, a0, a1, a2, a3, xh.x, xh.y);
      const float2 dl = ldsf2(dsc + ((2 * il) * 16 + 8 * hf) * 4);
      const float2 dh = ldsf2(dsc + ((2 * il + 1) * 16 + 8 * hf) * 4);
      u[2 * hf] = fmaf(magic_f(Dl[0] * sl), dl.x, u[2 * hf]);   // |dot * sc| <= 32*15*127*63 < 2^22
      u[2 * hf + 1] = fmaf(magic_f(Dl[1] * sl), dl.y, u[2 * hf + 1]);
      u[2 * hf] = fmaf(magic_f(Dh[2] * sh), dh.x, u[2 * hf]);
      u[2 * hf + 1] = fmaf(magic_f(Dh[3] * sh), dh.y, u[2 * hf + 1]);
    }
  }
  // min term: [rows x 8 sub-blocks] (mins 0..63, exact in tf32) x [8 sub-blocks x tokens] (d8 * block sum, hi + lo)
  const uint32_t m0 = __float_as_uint((float)byte_of(mn[0], t)), m1 = __float_as_uint((float)byte_of(mn[1], t));
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h.x));   // {d, dmin} of row g
#pragma unroll
  for (int hf = 0; hf < NH; ++hf) {
    const float z0 = ldsf(A.sZ + (((uint32_t)b0 + t) * 16u + 8u * hf + g) * 4u);
    const float z1 = ldsf(A.sZ + (((uint32_t)b0 + t + 4) * 16u + 8u * hf + g) * 4u);
    const uint32_t h0 = __float_as_uint(z0) & 0xFFFFE000u, h1 = __float_as_uint(z1) & 0xFFFFE000u;
    float dm[4] = {0.f, 0.f, 0.f, 0.f};
    mma_tf32_k8(dm, m0, 0u, m1, 0u, h0, h1);
    mma_tf32_k8(dm, m0, 0u, m1, 0u, __float_as_uint(z0 - __uint_as_float(h0)), __float_as_uint(z1 - __uint_as_float(h1)));
    acc[2 * hf] += dd.x * u[2 * hf] - dd.y * dm[0];
    acc[2 * hf + 1] += dd.x * u[2 * hf + 1] - dd.y * dm[1];
  }
}

// ---------------------------------------------------------------------------------------------- Q6_K unit
// 16-weight scale groups: A rows 0-7 carry group s=0 of a 32-block in the first 16 k slots, rows 8-15 group s=1 in the
// last 16 (zeros elsewhere), so one m16n8k32 against the block's activations yields both groups' dots.  Group (ip, q4, s) holds weights 128ip + 32q4 + 16s + 4t.. of the
// super-block: low nibbles from ql[64ip + 32(q4&1) + 16s + 4t] >> 4(q4>>1), two high bits from
// qh[32ip + 16s + 4t] >> 2q4.  The two groups share the activation scale, so their scaled dots are added as
// integers before the conversion (|sum| < 2^24).
// Four 6-bit codes -> four int8 values 4*(code - 32): the code sits in bits 2..7 of its byte with its top bit flipped,
// which is the two's-complement byte of 4*(code - 32) (range -128..124).  The factor 4 is taken out again through d.
__device__ __forceinline__ uint32_t unpack6_tl(uint32_t qlw, uint32_t qhw, int q4) {
  const uint32_t lo = q4 >> 1 ? qlw >> 2 : qlw << 2;                                          // nibble -> bits 2..5
  const uint32_t hi = q4 == 0 ? qhw << 6 : (q4 == 1 ? qhw << 4 : (q4 == 2 ? qhw << 2 : qhw));  // 2 bits -> bits 6, 7
  return (lo & 0x3C3C3C3Cu) | ((hi & 0xC0C0C0C0u) ^ 0x80808080u);
}

template <int NH, int AL>
__device__ __forceinline__ void unit_q6k(uint32_t pg, int b0, const TileView& A, int g, int t, float (&acc)[4]) {
  uint32_t sc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) sc[i] = lds32_h<AL>(pg + 192 + 4 * i);
  float u[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t tok = A.sA + (uint32_t)g * A.a_stride + (uint32_t)b0 * 32u + 4u * (uint32_t)t;
  const uint32_t dsc = A.sD + ((uint32_t)b0 * 16u + 2u * (uint32_t)t) * 4u;
#pragma unroll
  for (int ip = 0; ip < 2; ++ip) {
    uint32_t ql[2][2], qh[2];   // [s][q4 & 1]
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      ql[s][0] = lds32_h<AL>(pg + 64 * ip + 16 * s + 4 * t);
      ql[s][1] = lds32_h<AL>(pg + 64 * ip + 32 + 16 * s + 4 * t);
      qh[s] = lds32_h<AL>(pg + 128 + 32 * ip + 16 * s + 4 * t);
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const int b = 4 * ip + q4, gi = 8 * ip + 2 * q4;
      const uint32_t a0 = unpack6_tl(ql[0][q4 & 1], qh[0], q4), a1 = unpack6_tl(ql[1][q4 & 1], qh[1], q4);
      const int s0 = sbyte_of(sc[gi >> 2], gi & 3), s1 = sbyte_of(sc[gi >> 2], (gi & 3) + 1);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        const uint32_t x0 = lds32(tok + hf * 8 * A.a_stride + b * 32);
        const uint32_t x1 = lds32(tok + hf * 8 * A.a_stride + b * 32 + 16);
        // one m16n8k32: rows 0-7 = group 0 in the first 16 k slots (zeros in the rest), rows 8-15 = group 1 in the last 16
        int D[4];
        mma_i8_k32(D, a0, 0u, 0u, a1, x0, x1);
        const float2 d8 = ldsf2(dsc + (b * 16 + 8 * hf) * 4);
        u[2 * hf] = fmaf((float)(D[0] * s0 + D[2] * s1), d8.x, u[2 * hf]);
        u[2 * hf + 1] = fmaf((float)(D[1] * s0 + D[3] * s1), d8.y, u[2 * hf + 1]);
      }
    }
  }
  const float d = 0.25f * __half2float(*reinterpret_cast<const __half*>(tl_smem + pg + 208));   // the weights carry a factor 4
#pragma unroll
  for (int i = 0; i < 2 * NH; ++i) acc[i] = fmaf(d, u[i], acc[i]);
}

// ---------------------------------------------------------------------------------------------- Q8_0 unit
// Eight consecutive 34-byte blocks (256 weights, 272 bytes; pg is 16-byte aligned).  The weights are int8 already:
// A rows 0-7 carry block 2i, rows 8-15 block 2i+1, one mma against the activations of each.  Inside a block the
// codes start at byte 2, so an even block's words straddle aligned words (funnel shift) and an odd block's are aligned.
template <int NH>
__device__ __forceinline__ void unit_q80(uint32_t pg, int b0, const TileView& A, int g, int t, float (&acc)[4]) {
  const uint32_t tok = A.sA + (uint32_t)g * A.a_stride + (uint32_t)b0 * 32u + 8u * (uint32_t)t;
  const uint32_t dsc = A.sD + ((uint32_t)b0 * 16u + 2u * (uint32_t)t) * 4u;
#pragma unroll
  for (int pr = 0; pr < 4; ++pr) {
    const uint32_t pe = pg + 68 * pr, po = pe + 34;        // even / odd block of the pair
    const uint32_t x0 = lds32(pe + 8 * t), x1 = lds32(pe + 8 * t + 4), x2 = lds32(pe + 8 * t + 8);
    const uint32_t a0 = __funnelshift_r(x0, x1, 16), a2 = __funnelshift_r(x1, x2, 16);
    const uint32_t a1 = lds32(po + 2 + 8 * t), a3 = lds32(po + 6 + 8 * t);
    const float de = __half2float(*reinterpret_cast<const __half*>(tl_smem + pe));
    const float d_odd = __half2float(*reinterpret_cast<const __half*>(tl_smem + po));
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      const uint2 xl = lds64(tok + hf * 8 * A.a_stride + (2 * pr) * 32);
      const uint2 xh = lds64(tok + hf * 8 * A.a_stride + (2 * pr + 1) * 32);
      int Dl[4], Dh[4];
      mma_i8_k32(Dl, a0, a1, a2, a3, xl.x, xl.y);
      mma_i8_k32(Dh, a0, a1, a2, a3, xh.x, xh.y);
      const float2 dl = ldsf2(dsc + ((2 * pr) * 16 + 8 * hf) * 4);
      const float2 dh = ldsf2(dsc + ((2 * pr + 1) * 16 + 8 * hf) * 4);
      acc[2 * hf] = fmaf((float)Dl[0], de * dl.x, acc[2 * hf]);
      acc[2 * hf + 1] = fmaf((float)Dl[1], de * dl.y, acc[2 * hf + 1]);
      acc[2 * hf] = fmaf((float)Dh[2], d_odd * dh.x, acc[2 * hf]);
      acc[2 * hf + 1] = fmaf((float)Dh[3], d_odd * dh.y, acc[2 * hf + 1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------- Q4_0 / IQ3_S units
// 32-weight sub-blocks with one scale each: sub-blocks 2i and 2i+1 of the unit share an mma (A rows 0-7 / 8-15), as
// for Q8_0.  A lane decodes only the eight weights it feeds (k = 8t..8t+7 of the sub-block, natural order).
// Contribution of a sub-block: wa * d8 * dot - wb * z (Q4_0: wa = d, wb = 8d, z = the fp16 raw block sum, as
// vecdotq.cuh:46-66; IQ3_S: wa = d*(0.5+s)*0.5, no second term, vecdotq.cuh IQ3_S path).
template <int QT>
__device__ __forceinline__ void decode_part(const uint8_t* u, int j, int t, const uint32_t* grid, uint32_t& w0, uint32_t& w1,
                                            float& wa, float& wb) {
  if constexpr (QT == KQ_TYPE_Q4_0) {
    const uint8_t* b = u + 18 * j;
    const float d = ld_h(b);
    const uint32_t q0 = ld_u16x2(b + 2 + 8 * (t & 1)), q1 = ld_u16x2(b + 6 + 8 * (t & 1));
    const int sh = (t >> 1) * 4;                       // lanes 2, 3 take the high nibbles (weights 16..31)
    w0 = (q0 >> sh) & 0x0F0F0F0Fu;
    w1 = (q1 >> sh) & 0x0F0F0F0Fu;
    wa = d; wb = 8.0f * d;
  } else {   // IQ3_S
    const float d = ld_h(u);
    const uint8_t* qs = u + 2 + 8 * j;
    const uint32_t qh = u[66 + j];
    const uint32_t i1 = qs[2 * t] | ((qh << (8 - 2 * t)) & 256u);
    const uint32_t i2 = qs[2 * t + 1] | ((qh << (7 - 2 * t)) & 256u);
    const uint32_t sg = u[74 + 4 * j + t];
    w0 = negate_bytes(grid[i1], nibble_to_bytemask(sg & 15u));
    w1 = negate_bytes(grid[i2], nibble_to_bytemask(sg >> 4));
    const uint32_t s4 = (u[106 + (j >> 1)] >> (4 * (j & 1))) & 15u;
    wa = d * (0.5f + (float)s4) * 0.5f; wb = 0.f;
  }
}

template <int QT, int NH>
__device__ __forceinline__ void unit_g32(uint32_t pg, int b0, const TileView& A, const uint32_t* grid, int g, int t,
                                         float (&acc)[4]) {
  const uint8_t* u = tl_smem + pg;
  const uint32_t tok = A.sA + (uint32_t)g * A.a_stride + (uint32_t)b0 * 32u + 8u * (uint32_t)t;
  const uint32_t dsc = A.sD + ((uint32_t)b0 * 16u + 2u * (uint32_t)t) * 4u;
  const uint32_t zsc = A.sZ + ((uint32_t)b0 * 16u + 2u * (uint32_t)t) * 4u;
#pragma unroll
  for (int pr = 0; pr < 4; ++pr) {
    uint32_t a0, a1, a2, a3;
    float wa0, wb0, wa1, wb1;
    decode_part<QT>(u, 2 * pr, t, grid, a0, a2, wa0, wb0);
    decode_part<QT>(u, 2 * pr + 1, t, grid, a1, a3, wa1, wb1);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      const uint2 xl = lds64(tok + hf * 8 * A.a_stride + (2 * pr) * 32);
      const uint2 xh = lds64(tok + hf * 8 * A.a_stride + (2 * pr + 1) * 32);
      int Dl[4], Dh[4];
      mma_i8_k32(Dl, a0, a1, a2, a3, xl.x, xl.y);
      mma_i8_k32(Dh, a0, a1, a2, a3, xh.x, xh.y);
      const float2 dl = ldsf2(dsc + ((2 * pr) * 16 + 8 * hf) * 4);
      const float2 dh = ldsf2(dsc + ((2 * pr + 1) * 16 + 8 * hf) * 4);
      acc[2 * hf] = fmaf((float)Dl[0], wa0 * dl.x, acc[2 * hf]);
      acc[2 * hf + 1] = fmaf((float)Dl[1], wa0 * dl.y, acc[2 * hf + 1]);
      acc[2 * hf] = fmaf((float)Dh[2], wa1 * dh.x, acc[2 * hf]);
      acc[2 * hf + 1] = fmaf((float)Dh[3], wa1 * dh.y, acc[2 * hf + 1]);
      if constexpr (QT == KQ_TYPE_Q4_0) {
        const float2 zl = ldsf2(zsc + ((2 * pr) * 16 + 8 * hf) * 4);
        const float2 zh = ldsf2(zsc + ((2 * pr + 1) * 16 + 8 * hf) * 4);
        acc[2 * hf] -= wb0 * zl.x + wb1 * zh.x;
        acc[2 * hf + 1] -= wb0 * zl.y + wb1 * zh.y;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- Q2_K unit
// 16-weight groups with their own 4-bit scale and min.  Per 32-weight sub-block ONE m16n8k32 mma: lanes t = 0, 1
// hold weights 0..15 (group 0) and feed A rows 0-7, lanes t = 2, 3 hold weights 16..31 (group 1) and feed rows
// 8-15; the other half of each lane's fragment is zero, so rows 0-7 of the result are the group-0 dots and rows
// 8-15 the group-1 dots.  y += d*sc*d8*dot - dmin*m*(d8 * group sum of the activation codes), vecdotq.cuh Q2_K path.
template <int NH>
__device__ __forceinline__ void unit_q2k(uint32_t pg, int b0, const TileView& A, int g, int t, float (&acc)[4]) {
  const uint8_t* u = tl_smem + pg;
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(u + 80));   // {d, dmin}
  const uint32_t tok = A.sA + (uint32_t)g * A.a_stride + (uint32_t)b0 * 32u + 8u * (uint32_t)t;
  const uint32_t dsc = A.sD + ((uint32_t)b0 * 16u + 2u * (uint32_t)t) * 4u;
  const uint32_t zsc = A.sZ + ((uint32_t)b0 * 32u + 2u * (uint32_t)t) * 4u;       // [2 per block][16 tokens]
  const bool lo_half = t < 2;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = j >> 2, jj = j & 3;
    const uint32_t w0 = (ld_u32(u + 16 + 32 * n + 8 * t) >> (2 * jj)) & 0x03030303u;
    const uint32_t w1 = (ld_u32(u + 16 + 32 * n + 8 * t + 4) >> (2 * jj)) & 0x03030303u;
    const uint32_t a0 = lo_half ? w0 : 0u, a2 = lo_half ? w1 : 0u, a1 = lo_half ? 0u : w0, a3 = lo_half ? 0u : w1;
    const uint32_t s0 = u[2 * j], s1 = u[2 * j + 1];
    const float wa0 = dd.x * (float)(s0 & 15u), wb0 = dd.y * (float)(s0 >> 4);
    const float wa1 = dd.x * (float)(s1 & 15u), wb1 = dd.y * (float)(s1 >> 4);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      const uint2 x = lds64(tok + hf * 8 * A.a_stride + j * 32);
      int D[4];
      mma_i8_k32(D, a0, a1, a2, a3, x.x, x.y);
      const float2 d8 = ldsf2(dsc + (j * 16 + 8 * hf) * 4);
      const float2 z0 = ldsf2(zsc + ((2 * j) * 16 + 8 * hf) * 4);
      const float2 z1 = ldsf2(zsc + ((2 * j + 1) * 16 + 8 * hf) * 4);
      acc[2 * hf] += d8.x * (wa0 * (float)D[0] + wa1 * (float)D[2]) - (wb0 * z0.x + wb1 * z1.x);
      acc[2 * hf + 1] += d8.y * (wa0 * (float)D[1] + wa1 * (float)D[3]) - (wb0 * z0.y + wb1 * z1.y);
    }
  }
}

// ---------------------------------------------------------------------------------------------- fused all-gather
// Called by ONE whole warp of every CTA once all of the CTA's output stores are done and fenced at system scope (CTAs
// without rows call it at once).  The CTA that arrives last advances the call's epoch, stores it into flag[slot][rank]
// of every rank (release, system scope) and waits - bounded - until every rank's flag shows the same call: when the
// kernel completes, this rank's [M, N] buffer holds all ranks' columns.  Same protocol and flag arrays as
// kq_p2p_allgather; only plain loads and stores touch peer memory.
constexpr long long TL_PEER_WAIT_LIMIT = 1ll << 32;
// two 16-bit outputs: a half word with all bits set (the arrival sentinel, a NaN) becomes the canonical NaN
__device__ __forceinline__ uint32_t not_sentinel2(uint32_t w) { return w ^ (__vcmpeq2(w, 0xFFFFFFFFu) & 0x80008000u); }
// one output of any type, same rule (ll = 0: unchanged)
template <typename OutT>
__device__ __forceinline__ OutT out_value(float v, int ll) {
  OutT o = from_f32<OutT>(v);
  if (ll) {
    if constexpr (sizeof(OutT) == 2) {
      unsigned short b = *reinterpret_cast<unsigned short*>(&o);
      if (b == 0xFFFFu) { b = 0x7FFFu; o = *reinterpret_cast<OutT*>(&b); }
    } else {
      unsigned int b = *reinterpret_cast<unsigned int*>(&o);
      if (b == 0xFFFFFFFFu) { b = 0x7FFFFFFFu; o = *reinterpret_cast<OutT*>(&b); }
    }
  }
  return o;
}   // a good two seconds: ranks may be skewed at their first call
__device__ __forceinline__ void gather_finish(const TileParams& p, int lane) {
  int last = 0;
  if (lane == 0) last = atomicAdd(p.g_done + p.g_slot, 1u) == gridDim.x - 1;
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  uint32_t e = 0;
  if (lane == 0) {
    __threadfence_system();   // every CTA fenced its stores before it counted itself
    p.g_done[p.g_slot] = 0;
    e = p.g_epoch[p.g_slot] + 1;
    p.g_epoch[p.g_slot] = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  if (lane < p.g_world)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[lane] + p.g_slot * 8 + p.g_rank), "r"(e) : "memory");
  if (lane < p.g_world) {
    const uint32_t* f = p.peer_flags[p.g_rank] + p.g_slot * 8 + lane;
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int32_t)(v - e) >= 0) break;
      __nanosleep(100);
      if (clock64() - t0 > TL_PEER_WAIT_LIMIT) { atomicExch(p.g_status, 16 + lane); break; }
    }
  }
}

// ---------------------------------------------------------------------------------------------- kernel
// The kernel's unit of K is 256 weights: a super-block of the K-quants, eight blocks of Q8_0.
template <int QT> struct TileUnit { static constexpr int BYTES = Fmt<QT>::BYTES * (256 / Fmt<QT>::BLK); };
// NH = 1: up to 8 tokens per pass, NH = 2: up to 16
template <int QT, int NH, typename OutT>
__global__ void __launch_bounds__(TL_THREADS, 1) gemv_tile_kernel(const TileParams p) {
  using F = Fmt<QT>;
  uint8_t* const smem = tl_smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + TL_HEADER - 8);
  uint32_t* s_grid = reinterpret_cast<uint32_t*>(smem + TL_HEADER);   // IQ3_S only
  uint8_t* sA = smem + TL_HEADER + (QT == KQ_TYPE_IQ3_S ? TL_GRID_BYTES : 0);
  float* sD = reinterpret_cast<float*>(sA + p.a_bytes);
  float* sZ = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sD) + p.d_bytes);
  float4* sRed = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(sZ) + p.z_bytes);   // [2][16 warps][32 lanes]
  float* sT = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sRed) + TL_NRED * TL_CW * 512);   // [16 tokens][12]: transpose tile
  uint8_t* ring = reinterpret_cast<uint8_t*>(sT) + TL_TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  const int ks = blockIdx.x % p.ks;
  const int grp = blockIdx.x / p.ks, ngrp = gridDim.x / p.ks;
  const int rt0 = (int)((int64_t)grp * p.ntiles / ngrp), rt1 = (int)((int64_t)(grp + 1) * p.ntiles / ngrp);
  pdl_trigger();
  if (p.g_reset != nullptr && warp == TL_CW) {
    // sentinel-polled gather: refill the buffer the producer of this call's activations has just consumed, so that its
    // next use starts from "nothing has arrived".  After the predecessor (that producer) has completed; before any of
    // this CTA's outputs, which is what lets a peer move on to the call that writes the buffer again.
    pdl_wait();
    const uint32_t a = (uint32_t)((uint64_t)blockIdx.x * p.g_reset_n / gridDim.x), b = (uint32_t)((uint64_t)(blockIdx.x + 1) * p.g_reset_n / gridDim.x);
    const uint4 ones = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    for (uint32_t i = a + lane; i < b; i += 32) p.g_reset[i] = ones;
    __threadfence();
  }
  if (rt0 >= rt1) {
    if (p.g_world > 1 && !p.g_ll && warp == 0) { pdl_wait(); gather_finish(p, lane); }
    return;
  }
  const int nst = rt1 - rt0;
  const int blk0 = (int)((int64_t)ks * p.nblk / p.ks), blk1 = (int)((int64_t)(ks + 1) * p.nblk / p.ks);
  const int nsb = blk1 - blk0;
  const uint32_t bar_full = s_u32(bars), bar_empty = s_u32(bars + TL_MAX_STAGES), bar_act = s_u32(bars + 2 * TL_MAX_STAGES);
  const uint32_t bar_rfull = s_u32(bars + 2 * TL_MAX_STAGES + 1), bar_rempty = s_u32(bars + 2 * TL_MAX_STAGES + 1 + TL_NRED);
  const uint32_t bar_fin = s_u32(bars + 2 * TL_MAX_STAGES + 1 + 2 * TL_NRED);   // split-K: the reducer has published this CTA's tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { bar_init(bar_full + 8 * s, 1); bar_init(bar_empty + 8 * s, TL_CW); }
    bar_init(bar_act, 1);
    for (int b = 0; b < TL_NRED; ++b) { bar_init(bar_rfull + 8 * b, TL_CW); bar_init(bar_rempty + 8 * b, 1); }
    bar_init(bar_fin, 1);
    *s_abort = 0;
    *reinterpret_cast<volatile int*>(smem + TL_HEADER - 16) = 0;   // consumer warps past the split-K finish (fused gather)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if constexpr (QT == KQ_TYPE_IQ3_S) {
    for (int i = threadIdx.x; i < 512; i += TL_THREADS) s_grid[i] = iq3s_expand(c_iq3s_codes_t[i], KQ_IQ3S_TOP);
  }
  __syncthreads();

  if (warp == TL_CW + 1) {
    // ------------------------------------------------------------------ producer
    const int k0 = blk0 * 256, klen = nsb * 256;
    const int b32_0 = k0 >> 5, nb32 = klen >> 5;
    const int tt = p.m0 >> 4;
    const int ntok = p.mcount < 8 * NH ? p.mcount : 8 * NH;
    const size_t seg0 = (size_t)blk0 * TileUnit<QT>::BYTES;
    const uint32_t seglen = (uint32_t)nsb * TileUnit<QT>::BYTES;
    const int contig = p.contig;
    int slot = 0;          // ring position of the next stage to issue
    uint32_t eph = 1;      // parity that shows the slot's previous contents consumed (passes at once on the first lap)
    // every window is rounded out to 16-byte units; the host passes only row counts whose byte size is a multiple of
    // 16 (and a 16-byte aligned base), so the rounding never reaches outside the tensor
    auto issue_stage = [&](int q) {
      const int row0 = (rt0 + q) * TL_ROWS;
      const uint32_t dst = s_u32(ring + (size_t)slot * p.stage_bytes);
      const uint32_t bar = bar_full + 8 * slot;
      if (contig) {
        if (lane == 0) {
          const int rows = (p.n - row0) < TL_ROWS ? (p.n - row0) : TL_ROWS;
          const uintptr_t ga = (uintptr_t)(p.W + (size_t)row0 * p.rowbytes);
          const CopyWindow cw = copy_window(ga, ga + (size_t)rows * p.rowbytes);
          bar_expect_tx(bar, cw.bulk);
          copy_g2s(dst, (const void*)cw.a0, cw.bulk, bar);
        }
      } else {
        CopyWindow cw;
        cw.a0 = 0; cw.lead = 0; cw.bulk = 0;
        const int row = row0 + lane;
        if (lane < TL_ROWS && row < p.n) {
          const uintptr_t ga = (uintptr_t)(p.W + (size_t)row * p.rowbytes + seg0);
          cw = copy_window(ga, ga + seglen);
        }
        uint32_t total = cw.bulk;
#pragma unroll
        for (int mask = 4; mask > 0; mask >>= 1) total += __shfl_xor_sync(0xffffffffu, total, mask);
        if (lane == 0) bar_expect_tx(bar, total);   // row0 < n, so total > 0
        __syncwarp();
        if (cw.bulk) copy_g2s(dst + (uint32_t)lane * p.row_stride, (const void*)cw.a0, cw.bulk, bar);
      }
      if (++slot == S) { slot = 0; eph ^= 1; }
    };
    int q = 0;
    for (; q < nst && q < p.prefetch; ++q) issue_stage(q);   // the weights do not depend on the previous kernel
    pdl_wait();
    {
      if (lane == 0) {
        uint32_t total = (uint32_t)ntok * klen + (uint32_t)nb32 * 64u;
        if (p.zT != nullptr) total += (uint32_t)nb32 * p.zpb * 64u;
        bar_expect_tx(bar_act, total);
      }
      __syncwarp();
      if (lane < ntok)
        copy_g2s(s_u32(sA + lane * p.a_stride), p.qs + (size_t)(p.m0 + lane) * p.kpad + k0, (uint32_t)klen, bar_act);
      if (lane == 16) copy_g2s(s_u32(sD), p.dT + ((size_t)tt * p.nb32tot + b32_0) * 16, (uint32_t)nb32 * 64u, bar_act);
      if (lane == 17 && p.zT != nullptr)
        copy_g2s(s_u32(sZ), p.zT + ((size_t)tt * p.nb32tot + b32_0) * p.zpb * 16, (uint32_t)nb32 * p.zpb * 64u, bar_act);
    }
    bool ok = true;
    for (; q < nst; ++q) {
      if (q >= S) ok = bar_wait<TL_SLEEP_P>(bar_empty + 8 * slot, eph, s_abort);
      if (!ok) break;
      issue_stage(q);
    }
    // copies still in flight must land before the CTA may exit: the last min(q, S) stages issued
    {
      const int pending = q < S ? q : S;
      int sl = slot;
      uint32_t fph = eph ^ 1u;   // parity of the fill most recently issued into slots below `slot`
      for (int i = 0; i < pending; ++i) {
        if (--sl < 0) { sl = S - 1; fph ^= 1u; }
        bar_wait(bar_full + 8 * sl, q <= S ? 0u : fph, s_abort);
      }
    }
    bar_wait(bar_act, 0, s_abort);
    if (!ok && lane == 0) atomicExch(p.status, 1);
    return;
  }

  if (warp == TL_CW) {
    // ------------------------------------------------------------------ reducer
    OutT* y = reinterpret_cast<OutT*>(p.y);
    const int g = lane >> 2, t = lane & 3;
    const int nks = p.ks;
    // 16-byte stores need 16-byte aligned rows of the output / of the partials
    // (with the fused all-gather the host has checked every rank's buffer and the column offset)
    const bool vec_y = (p.g_world > 1 || ((uintptr_t)p.y % 16) == 0) && ((p.stride_y * sizeof(OutT)) % 16) == 0 &&
                       (((size_t)p.m0 * p.stride_y * sizeof(OutT)) % 16) == 0;
    const bool vec_part = (p.n % 4) == 0;
    for (int q = 0; q < nst; ++q) {
      const int buf = q & (TL_NRED - 1);
      if (!bar_wait<TL_SLEEP_R>(bar_rfull + 8 * buf, (uint32_t)((q / TL_NRED) & 1), s_abort)) { if (lane == 0) atomicExch(p.status, 5); return; }
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < TL_CW; ++w) {
        const float4 v = sRed[(buf * TL_CW + w) * 32 + lane];
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      }
      __syncwarp();
      if (lane == 0) bar_arrive(bar_rempty + 8 * buf);
      const int row0 = (rt0 + q) * TL_ROWS;
      const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
      // Transpose through a small shared tile so that one lane stores the 8 rows of one token with a 16-byte store
      // (two for fp32): value (row g, token tl) -> sT[tl][g], row stride 12 floats (conflict-free).  The scattered
      // 2-byte stores this replaces cost 1.6 us (8 tokens) to 4.4 us (16 tokens) of a 17408x5120 call.
      __syncwarp();   // the previous stage's tile has been read
#pragma unroll
      for (int i = 0; i < 2 * NH; ++i) sT[(2 * t + (i & 1) + 8 * (i >> 1)) * 12 + g] = vals[i];
      __syncwarp();
      if (lane < p.mcount && row0 < p.n) {
        const int tl = lane;
        const float4 va = *reinterpret_cast<const float4*>(sT + tl * 12), vb = *reinterpret_cast<const float4*>(sT + tl * 12 + 4);
        const float v8[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
        const bool whole = row0 + 8 <= p.n;
        if (nks > 1) {
          float* dst = p.part + ((size_t)ks * 16 + tl) * p.n + row0;   // published after the loop
          if (whole && vec_part) { __stcg(reinterpret_cast<float4*>(dst), va); __stcg(reinterpret_cast<float4*>(dst) + 1, vb); }
          else for (int i = 0; i < 8; ++i) if (row0 + i < p.n) __stcg(dst + i, v8[i]);
        } else {
          const int nd = p.g_world > 1 ? p.g_world : 1;
          for (int r = 0; r < nd; ++r) {   // fused all-gather: the same 16 bytes to every rank's buffer
            OutT* base = p.g_world > 1 ? reinterpret_cast<OutT*>(p.peer_y[r]) + p.g_col0 : y;
            OutT* dst = base + (size_t)(p.m0 + tl) * p.stride_y + row0;
            if (whole && vec_y) {
              if constexpr (sizeof(OutT) == 4) {
                if (p.g_ll) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) reinterpret_cast<float*>(dst)[i] = out_value<float>(v8[i], 1);
                } else {
                  reinterpret_cast<float4*>(dst)[0] = va; reinterpret_cast<float4*>(dst)[1] = vb;
                }
              } else {
                OutT o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = from_f32<OutT>(v8[i]);
                uint4 w = *reinterpret_cast<const uint4*>(o);
                if (p.g_ll) { w.x = not_sentinel2(w.x); w.y = not_sentinel2(w.y); w.z = not_sentinel2(w.z); w.w = not_sentinel2(w.w); }
                *reinterpret_cast<uint4*>(dst) = w;
              }
            } else {
              for (int i = 0; i < 8; ++i) if (row0 + i < p.n) dst[i] = out_value<OutT>(v8[i], p.g_ll);
            }
          }
        }
      }
    }
    if (nks == 1 && p.g_world > 1 && !p.g_ll) {
      __threadfence_system();   // this warp issued all of the CTA's output stores
      __syncwarp();
      gather_finish(p, lane);
    }
    if (nks > 1) {
      // one fence and one round of counter updates for all tiles of this CTA.  The split that arrives last at a
      // tile's counter finishes the tile; the list of those tiles goes to the consumer warps (idle by now),
      // which finish them in parallel.  The partial tiles' buffers are free: every consumer is past its last stage.
      uint8_t* s_last = reinterpret_cast<uint8_t*>(sRed);
      __threadfence();
      __syncwarp();
      for (int idx = lane; idx < nst; idx += 32) s_last[idx] = atomicAdd(p.cnt + rt0 + idx, 1) == nks - 1;
      __threadfence();
      __syncwarp();
      if (lane == 0) bar_arrive(bar_fin);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  if (!bar_wait(bar_act, 0, s_abort)) { if (lane == 0) atomicExch(p.status, 2); return; }
  const TileView A{(uint32_t)(sA - smem), (uint32_t)p.a_stride, (uint32_t)(reinterpret_cast<uint8_t*>(sD) - smem),
                   (uint32_t)(reinterpret_cast<uint8_t*>(sZ) - smem)};
  const int g = lane >> 2, t = lane & 3;
  const int contig = p.contig;
  const uint32_t row_stride = contig ? (uint32_t)p.rowbytes : (uint32_t)p.row_stride;
  const uint32_t stage_bytes = (uint32_t)p.stage_bytes, ring_a = (uint32_t)(ring - smem);
  const bool rows_same_parity = (p.rowbytes & 3) == 0 && (row_stride & 3u) == 0;   // all rows of a stage equally aligned mod 4
  // row r of a stage starts at r * row_stride + the low four bits of its global address
  const uint32_t off_base = (uint32_t)(((uintptr_t)p.W + (size_t)blk0 * TileUnit<QT>::BYTES) & 15);
  const uint32_t row_step = (uint32_t)(p.rowbytes & 15);
  int first = warp;   // first super-block of the current stage that belongs to this warp
  int slot = 0;
  uint32_t fph = 0;
  for (int q = 0; q < nst; ++q) {
    const int buf = q & (TL_NRED - 1);
    if (!bar_wait<TL_SLEEP_C>(bar_full + 8 * slot, fph, s_abort)) { if (lane == 0) atomicExch(p.status, 3); return; }
    const uint32_t row0 = (uint32_t)(rt0 + q) * TL_ROWS;
    const uint32_t lowbits = contig ? (off_base + row0 * row_step) & 15u : (off_base + (row0 + g) * row_step) & 15u;
    const uint32_t rg = ring_a + (uint32_t)slot * stage_bytes + (uint32_t)g * row_stride + lowbits;   // row g of the stage
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int sbi = first;
    for (; sbi < nsb; sbi += TL_CW) {
      const uint32_t pg = rg + (uint32_t)sbi * TileUnit<QT>::BYTES;
      if constexpr (QT == KQ_TYPE_Q4_K) unit_q4k<NH>(pg, sbi * 8, A, g, t, acc);
      if constexpr (QT == KQ_TYPE_Q8_0) unit_q80<NH>(pg, sbi * 8, A, g, t, acc);
      if constexpr (QT == KQ_TYPE_Q4_0 || QT == KQ_TYPE_IQ3_S) unit_g32<QT, NH>(pg, sbi * 8, A, s_grid, g, t, acc);
      if constexpr (QT == KQ_TYPE_Q2_K) unit_q2k<NH>(pg, sbi * 8, A, g, t, acc);
      if constexpr (QT == KQ_TYPE_Q6_K) {
        // every branch here is taken by all 32 lanes alike (the units contain warp-wide mma instructions)
        if (!rows_same_parity) unit_q6k<NH, 2>(pg, sbi * 8, A, g, t, acc);
        else if (pg & 2) unit_q6k<NH, 1>(pg, sbi * 8, A, g, t, acc);
        else unit_q6k<NH, 0>(pg, sbi * 8, A, g, t, acc);
      }
    }
    first = sbi - nsb;   // (q * nsb + sbi) % 16 == warp carries over to the next stage
    __syncwarp();
    if (lane == 0) bar_arrive(bar_empty + 8 * slot);
    if (++slot == S) { slot = 0; fph ^= 1u; }
    if (q >= TL_NRED && !bar_wait<TL_SLEEP_C>(bar_rempty + 8 * buf, (uint32_t)(((q / TL_NRED) - 1) & 1), s_abort)) {
      if (lane == 0) atomicExch(p.status, 4);
      return;
    }
    sRed[(buf * TL_CW + warp) * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncwarp();
    if (lane == 0) bar_arrive(bar_rfull + 8 * buf);
  }
  if (p.ks > 1) {
    // split-K finish: add the splits' partials in split order (deterministic) for the tiles this CTA completed
    if (!bar_wait(bar_fin, 0, s_abort)) { if (lane == 0) atomicExch(p.status, 6); return; }
    const uint8_t* s_last = reinterpret_cast<const uint8_t*>(sRed);
    OutT* y = reinterpret_cast<OutT*>(p.y);
    const int nks = p.ks;
    for (int idx = warp; idx < nst; idx += TL_CW) {
      if (!s_last[idx]) continue;
      const int rt = rt0 + idx, row0 = rt * TL_ROWS;
#pragma unroll
      for (int i = 0; i < 2 * NH; ++i) {
        const int row = row0 + g, tl = 2 * t + (i & 1) + 8 * (i >> 1);
        if (row < p.n && tl < p.mcount) {
          float v[4];
#pragma unroll
          for (int sp = 0; sp < 4; ++sp) v[sp] = sp < nks ? __ldcg(p.part + ((size_t)sp * 16 + tl) * p.n + row) : 0.f;
          float tot = v[0];
#pragma unroll
          for (int sp = 1; sp < 4; ++sp) if (sp < nks) tot += v[sp];
          const OutT o = out_value<OutT>(tot, p.g_ll);
          if (p.g_world > 1) {
            for (int r = 0; r < p.g_world; ++r)
              (reinterpret_cast<OutT*>(p.peer_y[r]) + p.g_col0)[(size_t)(p.m0 + tl) * p.stride_y + row] = o;
          } else {
            y[(size_t)(p.m0 + tl) * p.stride_y + row] = o;
          }
        }
      }
      if (lane == 0) p.cnt[rt] = 0;   // ready for the next launch on this scratch
    }
    if (p.g_world > 1 && !p.g_ll) {
      // the consumer warps issued this CTA's output stores: the last of them to get here hands the CTA over
      int* s_warps = reinterpret_cast<int*>(smem + TL_HEADER - 16);
      __threadfence_system();
      __syncwarp();
      int mine_last = 0;
      if (lane == 0) mine_last = atomicAdd(s_warps, 1) == TL_CW - 1;
      if (__shfl_sync(0xffffffffu, mine_last, 0)) gather_finish(p, lane);
    }
  }
}

// smallest K split whose activation slice leaves room for a ring of >= 4 stages
bool make_tile_config(int type, int64_t n, int64_t k, int mtok, TileConfig& c) {
  int blk, bytes;
  if (!type_is_core(type) || !type_geometry(type, &blk, &bytes)) return false;
  if (k % 256) return false;
  bytes *= 256 / blk;   // the kernel's unit of K is 256 weights
  blk = 256;
  const int nblk = (int)(k / blk);
  const int64_t rowbytes = (int64_t)nblk * bytes;
  const int sms = sm_count();
  const int seg_mode = options().tile_segments;   // 1: row segments even when the slice is the whole row
  for (int ks = 1; ks <= 4; ks *= 2) {
    if (nblk < ks) break;
    const int grid = sms / ks * ks;
    const int nsb = (nblk + ks - 1) / ks;
    const int klen = nsb * blk;
    const int contig = (ks == 1 && !seg_mode) ? 1 : 0;
    const int resid = type == KQ_TYPE_Q6_K ? 16 : 32;   // row stride mod 128: spreads the 8 rows over the banks
    int row_stride = (int)rowbytes;
    int stage_bytes;
    if (contig) {
      stage_bytes = (int)((TL_ROWS * rowbytes + 16 + 127) / 128 * 128);
    } else {
      row_stride = ((nsb * bytes + 16 + 15) / 16) * 16;
      while (row_stride % 128 != resid) row_stride += 16;
      stage_bytes = (TL_ROWS * row_stride + 127) / 128 * 128;
    }
    const int a_stride = klen + resid;
    const int a_bytes = (mtok * a_stride + 127) / 128 * 128;
    const int d_bytes = ((klen / 32) * 64 + 127) / 128 * 128;
    const int z_bytes = (type == KQ_TYPE_Q4_K || type == KQ_TYPE_Q4_0) ? d_bytes : (type == KQ_TYPE_Q2_K ? 2 * d_bytes : 0);
    const int fixed = TL_HEADER + (type == KQ_TYPE_IQ3_S ? TL_GRID_BYTES : 0) + a_bytes + d_bytes + z_bytes + TL_NRED * TL_CW * 512 + TL_TILE_BYTES;
    int stages = (TL_SMEM_LIMIT - fixed) / stage_bytes;
    if (stages > TL_MAX_STAGES) stages = TL_MAX_STAGES;
    // two whole-row stages of >= 32 KB keep more bytes in flight, in far larger requests, than a split over K whose stages
    // are row segments of a few KB (option tile_two_stage)
    const bool two_ok = options().tile_two_stage && contig && stages == 2 && stage_bytes >= 32768;
    if (stages < 3 && !two_ok) continue;
    if (ks > 1 && (int64_t)(n + TL_ROWS - 1) / TL_ROWS / (grid / ks) + 1 > TL_NRED * TL_CW * 512) continue;   // finish list
    if (ks > 1 && (n + TL_ROWS - 1) / TL_ROWS > KQ_CNT_SLOTS) continue;   // one arrival counter per 8-row tile
    if (stages < 4 && ks < 4 && nblk >= 2 * ks && !two_ok) continue;   // a deeper ring with a finer split is better
    c.ks = ks; c.grid = grid; c.stages = stages; c.row_stride = row_stride; c.stage_bytes = stage_bytes; c.contig = contig;
    c.a_stride = a_stride; c.a_bytes = a_bytes; c.d_bytes = d_bytes; c.z_bytes = z_bytes;
    c.smem = fixed + stages * stage_bytes;
    return true;
  }
  return false;
}

template <int QT, int NH, typename OutT>
int launch_tile(const TileParams& p, const TileConfig& c, cudaStream_t st) {
  auto kern = gemv_tile_kernel<QT, NH, OutT>;
  static DeviceOnce configured;   // the attribute belongs to the (function, device) pair
  if (configured.first_time()) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TL_SMEM_LIMIT));
    configured.done();
  }
  KQ_CUDA_TRY(launch_pdl(kern, dim3(c.grid), dim3(TL_THREADS), (size_t)c.smem, st, options().pdl != 0, p));
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

template <int QT>
int launch_tile_typed(const TileParams& p, const TileConfig& c, int nh, int y_dtype, cudaStream_t st) {
  switch (y_dtype) {
    case KQ_F32: return nh == 2 ? launch_tile<QT, 2, float>(p, c, st) : launch_tile<QT, 1, float>(p, c, st);
    case KQ_F16: return nh == 2 ? launch_tile<QT, 2, __half>(p, c, st) : launch_tile<QT, 1, __half>(p, c, st);
    case KQ_BF16: return nh == 2 ? launch_tile<QT, 2, __nv_bfloat16>(p, c, st) : launch_tile<QT, 1, __nv_bfloat16>(p, c, st);
  }
  set_error("unsupported output dtype %d", y_dtype);
  return KQ_EUNSUPPORTED;
}

}  // namespace

bool gemv_tile_supported(const void* W, int type, int64_t n, int64_t k, int mtok) {
  if ((uintptr_t)W % 2) return false;
  TileConfig c;
  return make_tile_config(type, n, k, mtok > 8 ? 16 : 8, c);
}

// K splits the shared-stage kernel would use for this shape (0 = shape not covered)
int gemv_tile_splits(int type, int64_t n, int64_t k, int mtok) {
  TileConfig c;
  return make_tile_config(type, n, k, mtok > 8 ? 16 : 8, c) ? c.ks : 0;
}

// one pass of up to 16 tokens starting at m0 (a multiple of 16)
int launch_gemv_tile(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m0, int mcount, void* y,
                     int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st, const GatherArgs* ga) {
  const int nh = mcount > 8 ? 2 : 1;
  TileConfig c;
  if (!make_tile_config(type, n, k, 8 * nh, c)) { set_error("tile GEMV: shape not covered"); return KQ_EUNSUPPORTED; }
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  TileParams p;
  p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.n = (int)n; p.nblk = (int)(k / 256); p.ks = c.ks;   // units of 256 weights
  p.ntiles = (int)((n + TL_ROWS - 1) / TL_ROWS); p.stages = c.stages; p.row_stride = c.row_stride;
  p.stage_bytes = c.stage_bytes; p.contig = c.contig; p.a_stride = c.a_stride; p.a_bytes = c.a_bytes;
  p.d_bytes = c.d_bytes; p.z_bytes = c.z_bytes; p.qs = P.qs; p.dT = P.dT;
  p.zT = type == KQ_TYPE_Q4_K ? (mmq ? P.zs8 : P.z32) : (type == KQ_TYPE_Q4_0 ? P.zs8 : (type == KQ_TYPE_Q2_K ? P.z16 : nullptr));
  p.zpb = type == KQ_TYPE_Q2_K ? 2 : 1;
  p.kpad = (int)P.kpad; p.nb32tot = (int)(P.kpad / 32); p.m0 = (int)m0; p.mcount = mcount;
  p.prefetch = options().pdl < c.stages ? options().pdl : c.stages;
  p.y = y; p.stride_y = stride_y; p.part = P.part; p.cnt = P.cnt; p.status = P.status;
  p.g_world = 0; p.g_slot = 0; p.g_rank = 0; p.g_col0 = 0; p.g_epoch = nullptr; p.g_done = nullptr; p.g_status = nullptr; p.g_ll = 0; p.g_reset = nullptr; p.g_reset_n = 0;
  for (int r = 0; r < 8; ++r) { p.peer_y[r] = nullptr; p.peer_flags[r] = nullptr; }
  if (ga && ga->world > 1) {
    p.g_world = ga->world; p.g_slot = ga->slot; p.g_rank = ga->rank; p.g_col0 = ga->col0;
    p.g_epoch = ga->epoch; p.g_done = ga->done; p.g_status = ga->status;
    p.g_ll = ga->ll; p.g_reset = (uint4*)ga->reset; p.g_reset_n = (uint32_t)(ga->reset_bytes / 16);
    for (int r = 0; r < ga->world; ++r) { p.peer_y[r] = ga->peer_y[r]; p.peer_flags[r] = ga->peer_flags[r]; }
    p.y = ga->peer_y[ga->rank];
  }
  switch (type) {
    case KQ_TYPE_Q4_K: return launch_tile_typed<KQ_TYPE_Q4_K>(p, c, nh, y_dtype, st);
    case KQ_TYPE_Q6_K: return launch_tile_typed<KQ_TYPE_Q6_K>(p, c, nh, y_dtype, st);
    case KQ_TYPE_Q4_0: return launch_tile_typed<KQ_TYPE_Q4_0>(p, c, nh, y_dtype, st);
    case KQ_TYPE_IQ3_S: return launch_tile_typed<KQ_TYPE_IQ3_S>(p, c, nh, y_dtype, st);
    case KQ_TYPE_Q2_K: return launch_tile_typed<KQ_TYPE_Q2_K>(p, c, nh, y_dtype, st);
    default: return launch_tile_typed<KQ_TYPE_Q8_0>(p, c, nh, y_dtype, st);
  }
}

}  // namespace kq
