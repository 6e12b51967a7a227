// Device helpers shared by the shared-stage decode kernels (kq_gemv_tile.cu, kq_gemv_kres.cu): mbarrier and bulk-copy
// wrappers with bounded waits, int8 / tf32 mma.sync wrappers, shared-memory loads by byte offset.
// Include inside an anonymous namespace of namespace kq.
#pragma once

constexpr uint32_t TL_MAGIC_I = 0x4B400000u;      // bits of 12582912.0f
constexpr float TL_MAGIC_F = 12582912.0f;
constexpr long long TL_WAIT_LIMIT = 1ll << 27;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(20000u)   // the thread may stay suspended this many ns before the test returns false
      : "memory");
  return ok != 0;
}
// bounded wait; SLEEP_NS between polls keeps a waiting warp out of the issue slots of the working ones
template <int SLEEP_NS = 64>
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (bar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (int it = 1;; ++it) {
    __nanosleep(SLEEP_NS);
    if (bar_try(bar, parity)) return true;
    if ((it & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > TL_WAIT_LIMIT) { *abort_flag = 1; return false; }
    }
  }
}
__device__ __forceinline__ void copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// tokens (A, 16 x 32 s8) x weights (B, 32 x 8 s8) -> s32
__device__ __forceinline__ void mma_i8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_i8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// d += A (16 x 8 tf32) x B (8 x 8 tf32)
__device__ __forceinline__ void mma_tf32_k8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float magic_f(int v) { return __int_as_float(v + (int)TL_MAGIC_I) - TL_MAGIC_F; }
__device__ __forceinline__ uint32_t byte_of(uint32_t w, int i) { return __byte_perm(w, 0u, 0x4440u | (uint32_t)i); }
__device__ __forceinline__ int sbyte_of(uint32_t w, int i) {   // sign-extended byte i in one permute
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"((uint32_t)i | ((8u | (uint32_t)i) * 0x1110u)));
  return (int)r;
}

// shared-memory loads by byte offset into the CTA's dynamic shared memory: ordinary loads (the compiler may
// schedule them around the arithmetic, but never across an mbarrier wait, which clobbers memory)
extern __shared__ __align__(128) uint8_t tl_smem[];
__device__ __forceinline__ uint32_t lds32(uint32_t a) { return *reinterpret_cast<const uint32_t*>(tl_smem + a); }
__device__ __forceinline__ uint2 lds64(uint32_t a) { return *reinterpret_cast<const uint2*>(tl_smem + a); }
__device__ __forceinline__ uint4 lds128(uint32_t a) { return *reinterpret_cast<const uint4*>(tl_smem + a); }
__device__ __forceinline__ float2 ldsf2(uint32_t a) { return *reinterpret_cast<const float2*>(tl_smem + a); }
__device__ __forceinline__ float ldsf(uint32_t a) { return *reinterpret_cast<const float*>(tl_smem + a); }
// 32 bits at a 2-byte aligned address.  AL = 0: the address is 4-byte aligned; 1: it is 2 mod 4; 2: either, decided
// per lane without a branch (the callers sit between warp-wide mma instructions and must not diverge)
template <int AL>
__device__ __forceinline__ uint32_t lds32_h(uint32_t a) {
  if constexpr (AL == 0) return lds32(a);
  else if constexpr (AL == 1) return __funnelshift_r(lds32(a - 2), lds32(a + 2), 16);
  else {
    const uint32_t b = a & ~3u;
    return __funnelshift_r(lds32(b), lds32(b + 4), (a & 2u) << 3);
  }
}

