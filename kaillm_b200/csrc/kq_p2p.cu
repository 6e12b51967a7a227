// All-gather of the ranks' output slices over NVLink by plain peer stores: every rank pushes its [M, N/G] slice into
// slot `rank` of every rank's gather buffer (the ranks' buffers are mapped into each other's address space by the
// caller, e.g. through torch symmetric memory), then raises a flag on every rank and waits until the flags of all
// ranks have reached the same call count.  One small kernel per call, no library collective:
//
//   copy     all CTAs: 16-byte loads of the local slice, one 16-byte store per destination rank (the local rank's
//            own buffer included); byte tail for sizes that are not a multiple of 16
//   publish  each CTA fences at system scope and counts itself done; the last CTA advances the call's epoch
//            (a device counter per flag slot, so a captured graph can be replayed) and stores it into
//            flag[slot][rank] of every rank (release, system scope)
//   wait     the last CTA's first `world` threads wait (acquire, system scope; sleeping between polls) until
//            flag[slot][r] >= epoch for every r, so when the kernel has completed the local gather buffer is whole
//
// The wait is bounded (2^32 clocks, a good two seconds - ranks of one job may be skewed by hundreds of milliseconds
// at their first call): on time-out the kernel writes a status word and returns with the gather buffer incomplete;
// the caller reads the word with its next synchronisation.  Only plain loads/stores touch peer memory (no TMA, no multicast).
// Buffer reuse: a rank may overwrite slot `rank` of a peer's buffer as soon as that peer has published the
// NEXT call on the same stream; a caller that alternates two buffers per stream is race-free.
#include "kq_common.cuh"

namespace kq {

namespace {

constexpr int P2P_MAX_RANKS = 8;
constexpr long long P2P_WAIT_LIMIT = 1ll << 32;

struct P2PParams {
  const uint8_t* src;
  size_t bytes;                       // of the whole slice (rows * row_bytes)
  size_t row_bytes;                   // bytes per row of the slice (== bytes for the rank-major layout)
  size_t dst_stride;                  // bytes between rows in the destination buffers
  size_t dst_off;                     // where this rank's first row starts in every destination buffer
  size_t src_stride;                  // bytes between rows of the source (row_bytes when the slice is contiguous)
  int skip_self;                      // the source IS this rank's columns of its own buffer: no store to itself
  uint8_t* dst[P2P_MAX_RANKS];        // each rank's gather buffer (world * bytes)
  uint32_t* flags[P2P_MAX_RANKS];     // each rank's flag array [slots][P2P_MAX_RANKS]
  uint32_t* epoch;                    // local: calls made so far per slot
  uint32_t* done;                     // local: CTAs finished per slot (returns to zero)
  int* status;
  int slot, rank, world;
  int vec16;                          // host-checked: src, every destination and the slice size are 16-byte aligned
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(1024) p2p_allgather_kernel(const P2PParams p) {
  const size_t nvec = p.bytes / 16;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
  // byte i of the slice = (row i / row_bytes, column i % row_bytes) -> dst_off + row * dst_stride + column
  if (p.vec16) {
    for (size_t i = tid; i < nvec; i += nthr) {
      const size_t b = i * 16, row = b / p.row_bytes, col = b - row * p.row_bytes;
      const uint4 v = *reinterpret_cast<const uint4*>(p.src + row * p.src_stride + col);
      for (int r = 0; r < p.world; ++r)
        if (!(p.skip_self && r == p.rank)) *reinterpret_cast<uint4*>(p.dst[r] + p.dst_off + row * p.dst_stride + col) = v;
    }
  } else {
    for (size_t i = tid; i < p.bytes; i += nthr) {
      const size_t row = i / p.row_bytes, col = i - row * p.row_bytes;
      const uint8_t v = p.src[row * p.src_stride + col];
      for (int r = 0; r < p.world; ++r)
        if (!(p.skip_self && r == p.rank)) p.dst[r][p.dst_off + row * p.dst_stride + col] = v;
    }
  }
  __syncthreads();
  if (gridDim.x > 1) {
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      __threadfence_system();   // this CTA's stores (ordered before by the barrier) are visible system-wide
      s_last = atomicAdd(p.done + p.slot, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
  }
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    __threadfence_system();   // every CTA's stores (ordered before by the barrier / the counter) are visible system-wide
    if (gridDim.x > 1) p.done[p.slot] = 0;
    const uint32_t e = p.epoch[p.slot] + 1;
    p.epoch[p.slot] = e;
    s_epoch = e;
  }
  __syncthreads();
  if ((int)threadIdx.x < p.world)   // one lane per destination: the flag stores travel in parallel
    st_release_sys(p.flags[threadIdx.x] + p.slot * P2P_MAX_RANKS + p.rank, s_epoch);
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    const uint32_t e = s_epoch;
    const uint32_t* f = p.flags[p.rank] + p.slot * P2P_MAX_RANKS + threadIdx.x;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(f) - e) < 0) {
      __nanosleep(100);
      if (clock64() - t0 > P2P_WAIT_LIMIT) { atomicExch(p.status, 1 + (int)threadIdx.x); break; }
    }
  }
}

}  // namespace

// rows == 0: the rank-major layout (the slice lands at rank * bytes of every buffer); rows > 0: the slice is
// [rows][row_bytes] and lands as columns rank * row_bytes .. of row-major buffers with row stride dst_stride
int launch_p2p_allgather(const void* src, size_t bytes, int64_t rows, size_t dst_stride, void* const* peer_dst,
                         uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* done, int slot, int rank, int world,
                         int* status, cudaStream_t st, size_t src_stride) {
  if (world < 1 || world > P2P_MAX_RANKS || rank < 0 || rank >= world || slot < 0) {
    set_error("kq_p2p_allgather: world %d (max %d), rank %d, slot %d", world, P2P_MAX_RANKS, rank, slot);
    return KQ_EINVAL;
  }
  if (bytes == 0) return KQ_OK;
  P2PParams p;
  p.src = (const uint8_t*)src; p.bytes = bytes; p.epoch = epoch; p.done = done; p.status = status;
  p.slot = slot; p.rank = rank; p.world = world;
  if (rows > 0) {
    if (bytes % (size_t)rows) { set_error("kq_p2p_allgather_2d: bytes is not a multiple of rows"); return KQ_EINVAL; }
    p.row_bytes = bytes / (size_t)rows; p.dst_stride = dst_stride; p.dst_off = (size_t)rank * p.row_bytes;
    if (dst_stride < (size_t)world * p.row_bytes) { set_error("kq_p2p_allgather_2d: destination row stride too small"); return KQ_EINVAL; }
  } else {
    p.row_bytes = bytes; p.dst_stride = 0; p.dst_off = (size_t)rank * bytes;
  }
  p.src_stride = src_stride ? src_stride : p.row_bytes;
  p.skip_self = rank < world && peer_dst[rank] && (const uint8_t*)src == (const uint8_t*)peer_dst[rank] + p.dst_off;
  // 16-byte stores: source, slice and row size, the strides and every buffer aligned
  uintptr_t bits = (uintptr_t)src | (uintptr_t)bytes | (uintptr_t)p.row_bytes | (uintptr_t)p.dst_stride | (uintptr_t)p.src_stride;
  for (int r = 0; r < P2P_MAX_RANKS; ++r) {
    p.dst[r] = r < world ? (uint8_t*)peer_dst[r] : nullptr;
    p.flags[r] = r < world ? peer_flags[r] : nullptr;
    if (r < world) {
      if (!peer_dst[r] || !peer_flags[r]) { set_error("kq_p2p_allgather: null buffer or flag pointer for rank %d", r); return KQ_EINVAL; }
      if ((uintptr_t)peer_flags[r] % 4) { set_error("kq_p2p_allgather: flag array of rank %d is not 4-byte aligned", r); return KQ_EINVAL; }
      bits |= (uintptr_t)peer_dst[r];
    }
  }
  p.vec16 = (bits & 15) == 0;   // otherwise every byte travels on its own (correct for any alignment, slow)
  // decode-sized slices (<= 256 KB) go through ONE CTA of 1024 threads: one system-scope fence and no CTA counter on
  // the way to the flags; larger ones use up to 32 CTAs
  size_t blocks = 1;
  unsigned threads = 1024;
  if (bytes > (256u << 10)) {
    threads = 256;
    blocks = (bytes / 16 + 255) / 256;
    if (blocks > 32) blocks = 32;
  }
  p2p_allgather_kernel<<<(unsigned)blocks, threads, 0, st>>>(p);
  options().launches += 1;
  KQ_CUDA_TRY(cudaGetLastError());
  return KQ_OK;
}

}  // namespace kq
