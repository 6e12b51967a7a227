// Decode GEMV for 3..16 tokens per pass with the activations resident in REGISTERS (Q4_K, Q6_K, Q8_0).
//
// Same skeleton as the shared-stage kernel of kq_gemv_tile.cu - persistent CTAs, a ring of stages of 8 weight rows x the
// CTA's K slice fed by bulk copies, consumer warps with int8 mma.sync, a reducer warp, optional split-K - but the K
// slice is dealt to the consumer warps ONCE: warp w owns the same few K units (64 weights of Q4_K, 128 of Q6_K, 64 of
// Q8_0) of every stage, loads the activation codes and scales of exactly those units from global memory into
// registers before its first stage, and from then on reads only weight bytes from shared memory.  In the shared-stage
// kernel every warp re-reads the activations of its unit for each group of 8 rows, which kept the shared-memory pipe
// busier than HBM (61 % against 45 % at 8 tokens); here a stage costs the weights' bytes once plus the partial tiles.
//
//   grid      one CTA per SM, in `ks` groups (group s = K slice s); ks is the smallest of 1, 2, 4 for which a warp's
//             share of the slice fits the registers set aside for it (PPW units per warp, cw consumer warps)
//   stage     8 consecutive weight rows x the K slice; one bulk copy when the slice is the whole row
//   consumer  lane (g, t): A-operand row g = weight row g of the stage, B-operand column g = token g (and g + 8); it ends
//             up with the outputs of row g for tokens 2t, 2t+1 (and 8 + 2t, 8 + 2t + 1), so it needs the block scales
//             of its own row only.  The Q4_K min term is a small tf32 GEMM per super-block, dealt to the warps
//             super-block by super-block.
//   reducer   adds the cw partial tiles of a stage in warp order (deterministic) and stores the outputs, or fp32
//             partials with ks > 1; the last split to arrive at a tile's counter adds the splits in split order
//
// The integer dots are exact; the fp32 combine follows vllm_gguf_plugin/csrc/gguf/vecdotq.cuh:328-379 (Q4_K),
// 447-491 (Q6_K), 165-177 (Q8_0).  All waits are bounded (see kq_tile_common.cuh).
#include "kq_common.cuh"

namespace kq {

namespace {

#include "kq_tile_common.cuh"

constexpr int KR_RG = 2;                       // groups of 8 rows per stage: two independent chains per warp and stage
constexpr int KR_ROWS = 8 * KR_RG;                   // rows per tile (= what a consumer warp does between two hand-overs)
constexpr int KR_SROWS = 8;                          // rows per ring slot (= one bulk copy): finer than a tile, so that
                                                     // the ring refills in small steps
constexpr int KR_HEADER = 1024;
constexpr int KR_TILE_BYTES = 1280;             // 16 x 20 floats
constexpr int KR_NRED = 2;
constexpr int KR_MAX_STAGES = 16;
constexpr int KR_SMEM_LIMIT = 232448;
constexpr int KR_SLEEP_C = 64, KR_SLEEP_R = 200, KR_SLEEP_P = 400;

struct KresParams {
  const uint8_t* W;
  int64_t rowbytes;
  int n, nblk, ks, ntiles;                 // nblk: 256-weight units per row
  int stages, row_stride, stage_bytes, contig, cw;
  const int8_t* qs;
  const float* dT;
  const float* zT;
  int kpad, nb32tot;
  int m0, mcount, prefetch;
  void* y;
  int y_dtype;
  int64_t stride_y;
  float* part;
  int* cnt;
  int* status;
};

struct KresConfig {
  int ks, grid, stages, row_stride, stage_bytes, contig, cw, ppw, smem;
};

__device__ __forceinline__ void store_y(void* y, int dt, size_t idx, float v) {
  if (dt == KQ_F32) reinterpret_cast<float*>(y)[idx] = v;
  else if (dt == KQ_F16) reinterpret_cast<__half*>(y)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
}

// two fp32 fused multiply-adds in one instruction (sm_100 packed fp32): c = a * b + c, lane-wise on (x, y)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(rc) : "l"(ra), "l"(rb));
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(rc));
  return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t ra, rb;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(ra) : "l"(rb));
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(ra));
  return r;
}
// exact int -> float for |v| < 2^22, two values: bits(12582912.0f) + v reinterpreted, minus 12582912.0f
__device__ __forceinline__ float2 magic2(int v0, int v1) {
  return add2(make_float2(__int_as_float(v0 + (int)TL_MAGIC_I), __int_as_float(v1 + (int)TL_MAGIC_I)),
              make_float2(-TL_MAGIC_F, -TL_MAGIC_F));
}

// ---------------------------------------------------------------------------------------------- per-format units
// A consumer warp owns ONE 256-weight unit (a super-block of the K-quants) of the CTA's K slice for the whole kernel:
// its index inside the unit is a compile-time constant everywhere, the unit's header is decoded once per stage, and
// the warp's share of the activations sits in registers: the codes always, the fp32 scales for up to 8 tokens (for
// 9..16 tokens the scales of the warp's unit live in a private 512-byte piece of shared memory, token-permuted so that
// one 16-byte load yields the two scales of both token halves).
template <int QT, int NH> struct Unit;

// Q4_K.  The 16 A rows of an m16n8k32 mma are the 8 weight rows twice: rows 0-7 carry the low nibbles of 32 bytes
// (sub-block 2il), rows 8-15 the high nibbles (sub-block 2il+1), so the unpacked words are the A fragment as they
// stand; one mma against the activations of each of the two sub-blocks, half of each result unused.  Inside a
// 32-block the k index is permuted (fragment k = 4t+i <-> position 8t+i, 16+4t+i <-> 8t+4+i) on both operands, so a
// lane's two activation registers of a sub-block are eight consecutive codes.
template <int NH> struct Unit<KQ_TYPE_Q4_K, NH> {
  static constexpr int SB_BYTES = 144;
  uint2 x[8][NH];                   // codes: sub-block j, token g + 8 hf, positions 8t..8t+7
  float2 d8[NH == 1 ? 8 : 1];       // NH == 1: scales of tokens 2t, 2t+1 per sub-block
  float z0[NH], z1[NH];             // min-term factors of sub-blocks t and t+4 for token g + 8 hf
  uint32_t sd;                      // NH == 2: byte offset of the warp's scale piece in shared memory

  // k0: first weight of the CTA's slice; sbi: this warp's unit in the slice; sd_off: the warp's 512-byte piece
  __device__ __forceinline__ void load(const KresParams& p, int k0, int sbi, uint32_t sd_off, int g, int t, int lane) {
    const int tt = p.m0 >> 4;
    const int b32 = (k0 >> 5) + sbi * 8;
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      const int tok = 8 * hf + g;
      const int8_t* src = p.qs + (size_t)(p.m0 + tok) * p.kpad + k0 + sbi * 256 + 8 * t;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        x[j][hf] = tok < p.mcount ? *reinterpret_cast<const uint2*>(src + 32 * j) : make_uint2(0u, 0u);
      const float* z = p.zT + ((size_t)tt * p.nb32tot + b32 + t) * 16 + tok;
      z0[hf] = z[0];
      z1[hf] = z[4 * 16];
    }
    const float* dsrc = p.dT + ((size_t)tt * p.nb32tot + b32) * 16;     // [8 sub-blocks][16 tokens]
    if constexpr (NH == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) d8[j] = *reinterpret_cast<const float2*>(dsrc + j * 16 + 2 * t);
      sd = 0;
    } else {
      // piece layout: [sub-block j][t][hf][2]: element (j, tok) goes to j*16 + (tok&7)/2*4 + (tok>>3)*2 + (tok&1)
      sd = sd_off;
      float* dst = reinterpret_cast<float*>(tl_smem + sd_off);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = lane + 32 * i, j = e >> 4, tok = e & 15;
        dst[j * 16 + ((tok & 7) >> 1) * 4 + (tok >> 3) * 2 + (tok & 1)] = dsrc[e];
      }
      __syncwarp();
    }
  }

  // pg: byte offset (in shared memory) of this warp's unit in row g of the stage's first row group; rs8: bytes between
  // row groups (8 rows).  acc[r][hf]: outputs of row 8r + g for tokens 2t, 2t+1 (+ 8 hf).
  __device__ __forceinline__ void run(uint32_t pg, uint32_t rs8, int t, float2 (&acc)[KR_RG][NH]) const {
    uint4 h[KR_RG];
    uint32_t sc[KR_RG][2];
    float2 u[KR_RG][NH];
#pragma unroll
    for (int r = 0; r < KR_RG; ++r) {
      h[r] = lds128(pg + r * rs8);   // {d, dmin}, scales[12]
      sc[r][0] = h[r].y & 0x3F3F3F3Fu;
      sc[r][1] = (h[r].w & 0x0F0F0F0Fu) | ((h[r].y >> 2) & 0x30303030u);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) u[r][hf] = make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int il = 0; il < 4; ++il) {
      float2 dl[NH], dh[NH];
      if constexpr (NH == 1) {
        dl[0] = d8[2 * il]; dh[0] = d8[2 * il + 1];
      } else {
        const uint4 ql = lds128(sd + ((2 * il) * 16 + 4 * t) * 4), qh = lds128(sd + ((2 * il + 1) * 16 + 4 * t) * 4);
        dl[0] = make_float2(__uint_as_float(ql.x), __uint_as_float(ql.y)); dl[NH - 1] = make_float2(__uint_as_float(ql.z), __uint_as_float(ql.w));
        dh[0] = make_float2(__uint_as_float(qh.x), __uint_as_float(qh.y)); dh[NH - 1] = make_float2(__uint_as_float(qh.z), __uint_as_float(qh.w));
      }
#pragma unroll
      for (int r = 0; r < KR_RG; ++r) {
        const uint2 w = lds64(pg + r * rs8 + 16 + 32 * il + 8 * t);
        const uint32_t a0 = w.x & 0x0F0F0F0Fu, a1 = (w.x >> 4) & 0x0F0F0F0Fu;
        const uint32_t a2 = w.y & 0x0F0F0F0Fu, a3 = (w.y >> 4) & 0x0F0F0F0Fu;
        const int sl = (int)byte_of(sc[r][il >> 1], (2 * il) & 3), sh = (int)byte_of(sc[r][il >> 1], (2 * il + 1) & 3);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          int Dl[4], Dh[4];
          mma_i8_k32(Dl, a0, a1, a2, a3, x[2 * il][hf].x, x[2 * il][hf].y);
          mma_i8_k32(Dh, a0, a1, a2, a3, x[2 * il + 1][hf].x, x[2 * il + 1][hf].y);
          u[r][hf] = fma2(magic2(Dl[0] * sl, Dl[1] * sl), dl[hf], u[r][hf]);   // |dot * sc| <= 32*15*127*63 < 2^22
          u[r][hf] = fma2(magic2(Dh[2] * sh, Dh[3] * sh), dh[hf], u[r][hf]);
        }
      }
    }
    // min term: [rows x 8 sub-blocks] (mins 0..63, exact in tf32) x [8 sub-blocks x tokens] (d8 * block sum - or the raw
    // fp16 block sum for the MMQ flavour - split hi + lo): two tf32 mmas per token half
#pragma unroll
    for (int r = 0; r < KR_RG; ++r) {
      const uint32_t mn0 = h[r].z & 0x3F3F3F3Fu, mn1 = ((h[r].w >> 4) & 0x0F0F0F0Fu) | ((h[r].z >> 2) & 0x30303030u);
      const uint32_t m0 = __float_as_uint((float)byte_of(mn0, t)), m1 = __float_as_uint((float)byte_of(mn1, t));
      const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&h[r].x));   // {d, dmin} of row g
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        const uint32_t h0 = __float_as_uint(z0[hf]) & 0xFFFFE000u, h1 = __float_as_uint(z1[hf]) & 0xFFFFE000u;
        float dm[4] = {0.f, 0.f, 0.f, 0.f};
        mma_tf32_k8(dm, m0, 0u, m1, 0u, h0, h1);
        mma_tf32_k8(dm, m0, 0u, m1, 0u, __float_as_uint(z0[hf] - __uint_as_float(h0)), __float_as_uint(z1[hf] - __uint_as_float(h1)));
        acc[r][hf] = fma2(make_float2(dd.x, dd.x), u[r][hf], make_float2(-dd.y * dm[0], -dd.y * dm[1]));
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------- kernel
template <int QT, int NH, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) gemv_kres_kernel(const KresParams p) {
  using U = Unit<QT, NH>;
  uint8_t* const smem = tl_smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + KR_HEADER - 8);
  const int CW = p.cw;
  constexpr int NV = KR_RG * NH / 2;                                    // float4 values per lane, warp and stage
  float4* sRed = reinterpret_cast<float4*>(smem + KR_HEADER);          // [KR_NRED][CW][NV][32 lanes]
  uint8_t* sScale = smem + KR_HEADER + KR_NRED * CW * NV * 512;         // [CW][512 bytes], 9..16 tokens only
  float* sT = reinterpret_cast<float*>(sScale + (NH == 2 ? CW * 512 : 0));   // [16 tokens][20]: the reducer's transpose tile
  uint8_t* ring = reinterpret_cast<uint8_t*>(sT) + KR_TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  const int ks = blockIdx.x % p.ks;
  const int grp = blockIdx.x / p.ks, ngrp = gridDim.x / p.ks;
  const int rt0 = (int)((int64_t)grp * p.ntiles / ngrp), rt1 = (int)((int64_t)(grp + 1) * p.ntiles / ngrp);
  pdl_trigger();
  if (rt0 >= rt1) return;
  const int nst = rt1 - rt0;
  const int blk0 = (int)((int64_t)ks * p.nblk / p.ks), blk1 = (int)((int64_t)(ks + 1) * p.nblk / p.ks);
  const int nsb = blk1 - blk0;                                          // <= CW
  const uint32_t bar_full = s_u32(bars), bar_empty = s_u32(bars + KR_MAX_STAGES);
  const uint32_t bar_rfull = s_u32(bars + 2 * KR_MAX_STAGES), bar_rempty = s_u32(bars + 2 * KR_MAX_STAGES + KR_NRED);
  const uint32_t bar_fin = s_u32(bars + 2 * KR_MAX_STAGES + 2 * KR_NRED);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { bar_init(bar_full + 8 * s, 1); bar_init(bar_empty + 8 * s, CW); }
    for (int b = 0; b < KR_NRED; ++b) { bar_init(bar_rfull + 8 * b, CW); bar_init(bar_rempty + 8 * b, 1); }
    bar_init(bar_fin, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp == CW + 1) {
    // ------------------------------------------------------------------ producer: weights only; it never waits for the
    // previous kernel (no kernel of this library writes weights), so its ring fills while that kernel drains
    const size_t seg0 = (size_t)blk0 * U::SB_BYTES;
    const uint32_t seglen = (uint32_t)nsb * U::SB_BYTES;
    const int contig = p.contig;
    int slot = 0;
    uint32_t eph = 1;
    auto issue_stage = [&](int q) {       // slot q = rows 8 (q & 1) .. of tile q >> 1
      const int row0 = (rt0 + (q >> 1)) * KR_ROWS + KR_SROWS * (q & 1);
      const uint32_t dst = s_u32(ring + (size_t)slot * p.stage_bytes);
      const uint32_t bar = bar_full + 8 * slot;
      if (contig) {
        if (lane == 0) {
          int rows = p.n - row0;
          rows = rows < 0 ? 0 : (rows < KR_SROWS ? rows : KR_SROWS);
          const uintptr_t ga = (uintptr_t)(p.W + (size_t)row0 * p.rowbytes);
          CopyWindow cw = copy_window(ga, ga + (size_t)rows * p.rowbytes);
          if (rows == 0) cw.bulk = 0;       // the second half of the last tile may be empty: the barrier still completes
          bar_expect_tx(bar, cw.bulk);
          if (cw.bulk) copy_g2s(dst, (const void*)cw.a0, cw.bulk, bar);
        }
      } else {
        CopyWindow cw;
        cw.a0 = 0; cw.lead = 0; cw.bulk = 0;
        const int row = row0 + lane;
        if (lane < KR_SROWS && row < p.n) {
          const uintptr_t ga = (uintptr_t)(p.W + (size_t)row * p.rowbytes + seg0);
          cw = copy_window(ga, ga + seglen);
        }
        uint32_t total = cw.bulk;
#pragma unroll
        for (int mask = 4; mask > 0; mask >>= 1) total += __shfl_xor_sync(0xffffffffu, total, mask);
        if (lane == 0) bar_expect_tx(bar, total);
        __syncwarp();
        if (cw.bulk) copy_g2s(dst + (uint32_t)lane * p.row_stride, (const void*)cw.a0, cw.bulk, bar);
      }
      if (++slot == S) { slot = 0; eph ^= 1; }
    };
    bool ok = true;
    int q = 0;
    for (; q < KR_RG * nst; ++q) {
      if (q >= S) ok = bar_wait<KR_SLEEP_P>(bar_empty + 8 * slot, eph, s_abort);
      if (!ok) break;
      issue_stage(q);
    }
    {   // copies still in flight must land before the CTA may exit: the last min(q, S) stages issued
      const int pending = q < S ? q : S;
      int sl = slot;
      uint32_t fph = eph ^ 1u;
      for (int i = 0; i < pending; ++i) {
        if (--sl < 0) { sl = S - 1; fph ^= 1u; }
        bar_wait(bar_full + 8 * sl, q <= S ? 0u : fph, s_abort);
      }
    }
    if (!ok && lane == 0) atomicExch(p.status, 1);
    return;
  }

  if (warp == CW) {
    // ------------------------------------------------------------------ reducer
    const int g = lane >> 2, t = lane & 3;
    const int nks = p.ks;
    // 16-byte stores need 16-byte aligned rows of the output / of the partials
    const int esz = p.y_dtype == KQ_F32 ? 4 : 2;
    const bool vec_y = ((uintptr_t)p.y % 16) == 0 && ((p.stride_y * esz) % 16) == 0 && (((size_t)p.m0 * p.stride_y * esz) % 16) == 0;
    const bool vec_part = (p.n % 4) == 0;
    pdl_wait();   // the outputs, partials and counters may still be in use by the previous kernel
    for (int q = 0; q < nst; ++q) {
      const int buf = q & (KR_NRED - 1);
      if (!bar_wait<KR_SLEEP_R>(bar_rfull + 8 * buf, (uint32_t)((q / KR_NRED) & 1), s_abort)) { if (lane == 0) atomicExch(p.status, 5); return; }
      // the partial tiles in warp order, eight loads in flight at a time (the warp count is a run-time value)
      float4 sum[NV];
#pragma unroll
      for (int e = 0; e < NV; ++e) sum[e] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        for (int w0 = 0; w0 < CW; w0 += 8) {
          float4 v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            v[i] = w0 + i < CW ? sRed[((buf * CW + w0 + i) * NV + e) * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int i = 0; i < 8; ++i) { sum[e].x += v[i].x; sum[e].y += v[i].y; sum[e].z += v[i].z; sum[e].w += v[i].w; }
        }
      }
      __syncwarp();
      if (lane == 0) bar_arrive(bar_rempty + 8 * buf);
      // Transpose through a small shared tile so that a lane stores 8 consecutive rows of one token with one or two
      // 16-byte stores: value (row 8r + g, token 2t + xy + 8hf) -> sT[token][row], row stride 20 floats (conflict-free).
      // Scattered 2-byte stores from this one warp cost 1.6 us (8 tokens) to 4.4 us (16 tokens) per 17408x5120 call.
      const int row0 = (rt0 + q) * KR_ROWS;
      __syncwarp();   // the previous stage's tile has been read by every lane
#pragma unroll
      for (int r = 0; r < KR_RG; ++r)
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
#pragma unroll
          for (int xy = 0; xy < 2; ++xy) {
            const int fi = (r * NH + hf) * 2 + xy;       // float index in the order the consumers packed them
            const float4 s4 = sum[fi >> 2];
            const float val = (fi & 3) == 0 ? s4.x : ((fi & 3) == 1 ? s4.y : ((fi & 3) == 2 ? s4.z : s4.w));
            sT[(2 * t + xy + 8 * hf) * 20 + 8 * r + g] = val;
          }
      __syncwarp();
      {
        const int tok = lane >> 1, rowv = row0 + 8 * (lane & 1);
        if (tok < p.mcount && rowv < p.n) {
          const float4 va = *reinterpret_cast<const float4*>(sT + tok * 20 + 8 * (lane & 1));
          const float4 vb = *reinterpret_cast<const float4*>(sT + tok * 20 + 8 * (lane & 1) + 4);
          const float v8[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
          const bool whole = rowv + 8 <= p.n;
          if (nks > 1) {
            float* dst = p.part + ((size_t)ks * 16 + tok) * p.n + rowv;
            if (whole && vec_part) { __stcg(reinterpret_cast<float4*>(dst), va); __stcg(reinterpret_cast<float4*>(dst) + 1, vb); }
            else for (int i = 0; i < 8; ++i) if (rowv + i < p.n) __stcg(dst + i, v8[i]);
          } else {
            const size_t idx = (size_t)(p.m0 + tok) * p.stride_y + rowv;
            if (whole && vec_y) {
              if (p.y_dtype == KQ_F32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + idx);
                dst[0] = va; dst[1] = vb;
              } else {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  if (p.y_dtype == KQ_F16) { const __half2 hh = __floats2half2_rn(v8[2 * i], v8[2 * i + 1]); w[i] = *reinterpret_cast<const uint32_t*>(&hh); }
                  else { const __nv_bfloat162 bb = __floats2bfloat162_rn(v8[2 * i], v8[2 * i + 1]); w[i] = *reinterpret_cast<const uint32_t*>(&bb); }
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.y) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
              for (int i = 0; i < 8; ++i) if (rowv + i < p.n) store_y(p.y, p.y_dtype, idx + i, v8[i]);
            }
          }
        }
      }
    }
    if (nks > 1) {
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
  const int g = lane >> 2, t = lane & 3;
  const bool mine = warp < nsb;          // a slice may have one unit fewer than there are consumer warps
  U res;
  pdl_wait();   // the quantized activations come from the kernel before this one
  if (mine) res.load(p, blk0 * 256, warp, (uint32_t)(sScale - smem) + (uint32_t)warp * 512u, g, t, lane);
  const int contig = p.contig;
  const uint32_t row_stride = contig ? (uint32_t)p.rowbytes : (uint32_t)p.row_stride;
  const uint32_t stage_bytes = (uint32_t)p.stage_bytes, ring_a = (uint32_t)(ring - smem);
  const uint32_t off_base = (uint32_t)(((uintptr_t)p.W + (size_t)blk0 * U::SB_BYTES) & 15);
  const uint32_t row_step = (uint32_t)(p.rowbytes & 15);
  const uint32_t unit_off = (uint32_t)warp * U::SB_BYTES;
  int slot = 0;
  uint32_t fph = 0;
  for (int q = 0; q < nst; ++q) {
    const int buf = q & (KR_NRED - 1);
    // a tile is KR_RG consecutive ring slots (the ring has an even number of slots, so they never wrap inside a tile)
#pragma unroll
    for (int r = 0; r < KR_RG; ++r)
      if (!bar_wait<KR_SLEEP_C>(bar_full + 8 * (slot + r), fph, s_abort)) { if (lane == 0) atomicExch(p.status, 3); return; }
    const uint32_t row0 = (uint32_t)(rt0 + q) * KR_ROWS;
    const uint32_t lowbits = contig ? (off_base + row0 * row_step) & 15u : (off_base + (row0 + g) * row_step) & 15u;
    const uint32_t pg = ring_a + (uint32_t)slot * stage_bytes + (uint32_t)g * row_stride + lowbits + unit_off;
    float2 acc[KR_RG][NH];
#pragma unroll
    for (int r = 0; r < KR_RG; ++r)
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) acc[r][hf] = make_float2(0.f, 0.f);
    if (mine) res.run(pg, stage_bytes, t, acc);   // the same branch for all 32 lanes; row group r sits in slot + r
    __syncwarp();
    if (lane < KR_RG) bar_arrive(bar_empty + 8 * (slot + lane));
    slot += KR_RG;
    if (slot == S) { slot = 0; fph ^= 1u; }
    if (q >= KR_NRED && !bar_wait<KR_SLEEP_C>(bar_rempty + 8 * buf, (uint32_t)(((q / KR_NRED) - 1) & 1), s_abort)) {
      if (lane == 0) atomicExch(p.status, 4);
      return;
    }
    {
      const float* af = reinterpret_cast<const float*>(&acc[0][0]);   // (r, hf, x/y) flat: 2 * KR_RG * NH floats
#pragma unroll
      for (int e = 0; e < NV; ++e)
        sRed[((buf * CW + warp) * NV + e) * 32 + lane] = make_float4(af[4 * e], af[4 * e + 1], af[4 * e + 2], af[4 * e + 3]);
    }
    __syncwarp();
    if (lane == 0) bar_arrive(bar_rfull + 8 * buf);
  }
  if (p.ks > 1) {
    // split-K finish: add the splits' partials in split order (deterministic) for the tiles this CTA completed
    if (!bar_wait(bar_fin, 0, s_abort)) { if (lane == 0) atomicExch(p.status, 6); return; }
    const uint8_t* s_last = reinterpret_cast<const uint8_t*>(sRed);
    const int nks = p.ks;
    for (int idx = warp; idx < nst; idx += CW) {
      if (!s_last[idx]) continue;
      const int rt = rt0 + idx, row0 = rt * KR_ROWS;
#pragma unroll
      for (int i = 0; i < 2 * NH * KR_RG; ++i) {
        const int row = row0 + 8 * (i / (2 * NH)) + g, tl = 2 * t + (i & 1) + 8 * ((i >> 1) % NH);
        if (row < p.n && tl < p.mcount) {
          float tot = __ldcg(p.part + ((size_t)0 * 16 + tl) * p.n + row);
          for (int sp = 1; sp < nks; ++sp) tot += __ldcg(p.part + ((size_t)sp * 16 + tl) * p.n + row);
          store_y(p.y, p.y_dtype, (size_t)(p.m0 + tl) * p.stride_y + row, tot);
        }
      }
      if (lane == 0) p.cnt[rt] = 0;   // ready for the next launch on this scratch
    }
  }
}

// ---------------------------------------------------------------------------------------------- host
// Two instantiations per format and token-half count.  An SM's registers are split over its four schedulers, so what
// a thread may use is set by the warps per scheduler: A = up to 16 warps in all (14 consumers, up to 128 registers),
// B = up to 24 warps (22 consumers, up to 80 registers).
constexpr int KR_MAXT_A = 16 * 32, KR_MAXT_B = 24 * 32;
constexpr int KR_CW_A = 14, KR_CW_B = 22, KR_CW_MIN = 10;

bool kres_type(int type) { return type == KQ_TYPE_Q4_K; }

// K split: the smallest of 1, 2, 4 whose slice has KR_CW_MIN..KR_CW_B units (one consumer warp per unit)
bool make_kres_config(int type, int64_t n, int64_t k, int nh, KresConfig& c) {
  if (!kres_type(type) || k % 256) return false;
  const int sb_bytes = 144;
  const int nblk = (int)(k / 256);
  const int64_t rowbytes = (int64_t)nblk * sb_bytes;
  const int sms = sm_count();
  for (int ks = 1; ks <= 4; ks *= 2) {
    if (nblk < ks) break;
    const int nsb = (nblk + ks - 1) / ks;          // the larger slices when nblk is not a multiple of ks
    if (nsb > KR_CW_B) continue;
    if (nsb < KR_CW_MIN) break;
    const int cw = nsb;
    const int grid = sms / ks * ks;
    const int contig = ks == 1 ? 1 : 0;
    int row_stride = (int)rowbytes, stage_bytes;
    if (contig) {
      stage_bytes = (int)((KR_SROWS * rowbytes + 16 + 127) / 128 * 128);
    } else {
      row_stride = ((nsb * sb_bytes + 16 + 15) / 16) * 16;
      while (row_stride % 128 != 32) row_stride += 16;   // spreads the 8 rows over the banks
      stage_bytes = (KR_SROWS * row_stride + 127) / 128 * 128;
    }
    const int nv = KR_RG * nh / 2;
    const int fixed = KR_HEADER + KR_NRED * cw * nv * 512 + (nh == 2 ? cw * 512 : 0) + KR_TILE_BYTES;
    int stages = (KR_SMEM_LIMIT - fixed) / stage_bytes;
    if (stages > KR_MAX_STAGES) stages = KR_MAX_STAGES;
    stages &= ~1;                                   // whole tiles of two slots
    if (stages < 4) continue;
    const int64_t tiles = (n + KR_ROWS - 1) / KR_ROWS;
    if (ks > 1 && (tiles / (grid / ks) + 1 > KR_NRED * cw * nv * 512 || tiles > KQ_CNT_SLOTS)) continue;
    c.ks = ks; c.grid = grid; c.stages = stages; c.row_stride = row_stride; c.stage_bytes = stage_bytes; c.contig = contig;
    c.cw = cw; c.ppw = 1; c.smem = fixed + stages * stage_bytes;
    return true;
  }
  return false;
}

template <int QT, int NH, bool B>
int launch_kres(const KresParams& p, const KresConfig& c, cudaStream_t st) {
  constexpr int MAXT = B ? KR_MAXT_B : KR_MAXT_A;
  auto kern = gemv_kres_kernel<QT, NH, MAXT>;
  static DeviceOnce configured;
  if (configured.first_time()) {
    KQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, KR_SMEM_LIMIT));
    configured.done();
  }
  KQ_CUDA_TRY(launch_pdl(kern, dim3(c.grid), dim3((c.cw + 2) * 32), (size_t)c.smem, st, options().pdl != 0, p));
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

}  // namespace

bool gemv_kres_supported(const void* W, int type, int64_t n, int64_t k, int mtok) {
  if ((uintptr_t)W % 16) return false;
  KresConfig c;
  return make_kres_config(type, n, k, mtok > 8 ? 2 : 1, c);
}

int gemv_kres_splits(int type, int64_t n, int64_t k, int mtok) {
  KresConfig c;
  return make_kres_config(type, n, k, mtok > 8 ? 2 : 1, c) ? c.ks : 0;
}

// one pass of up to 16 tokens starting at m0 (a multiple of 16)
int launch_gemv_kres(const void* W, int type, int64_t n, int64_t k, const Q8Ptrs& P, int64_t m0, int mcount, void* y,
                     int y_dtype, int64_t stride_y, bool mmq, cudaStream_t st) {
  const int nh = mcount > 8 ? 2 : 1;
  KresConfig c;
  if (!make_kres_config(type, n, k, nh, c)) { set_error("register-resident GEMV: shape not covered"); return KQ_EUNSUPPORTED; }
  int blk, bytes;
  type_geometry(type, &blk, &bytes);
  KresParams p;
  p.W = (const uint8_t*)W; p.rowbytes = k / blk * bytes; p.n = (int)n; p.nblk = (int)(k / 256); p.ks = c.ks;
  p.ntiles = (int)((n + KR_ROWS - 1) / KR_ROWS); p.stages = c.stages; p.row_stride = c.row_stride;
  p.stage_bytes = c.stage_bytes; p.contig = c.contig; p.cw = c.cw; p.qs = P.qs; p.dT = P.dT;
  p.zT = type == KQ_TYPE_Q4_K ? (mmq ? P.zs8 : P.z32) : nullptr;
  p.kpad = (int)P.kpad; p.nb32tot = (int)(P.kpad / 32); p.m0 = (int)m0; p.mcount = mcount;
  p.prefetch = 0;
  p.y = y; p.y_dtype = y_dtype; p.stride_y = stride_y; p.part = P.part; p.cnt = P.cnt; p.status = P.status;
  const bool b = c.cw > KR_CW_A;
  switch (type) {
    case KQ_TYPE_Q4_K:
      if (nh == 1) return b ? launch_kres<KQ_TYPE_Q4_K, 1, true>(p, c, st) : launch_kres<KQ_TYPE_Q4_K, 1, false>(p, c, st);
      return b ? launch_kres<KQ_TYPE_Q4_K, 2, true>(p, c, st) : launch_kres<KQ_TYPE_Q4_K, 2, false>(p, c, st);
  }
  set_error("register-resident GEMV: type %d not covered", type);
  return KQ_EUNSUPPORTED;
}

}  // namespace kq
