// Blackwell (sm_100a) primitives used by the tcgen05 kernels: mbarriers with bounded waits, TMA tile
// loads, TMEM allocation, UMMA shared-memory / instruction descriptors, tcgen05.mma issue and the
// TMEM -> register loads.  Everything is cta_group::1; every CTA issues its own TMA loads.
//
// Shared-memory operand tiles use the 128-byte swizzle: a tile is a stack of rows of 128 bytes
// (64 bf16), 8 rows form a 1024-byte atom, and the 16-byte piece `c` of row `r` lives at piece
// `c ^ (r & 7)`.  TMA (SWIZZLE_128B) writes that layout, the UMMA descriptors below read it, and
// sw128_offset() lets ordinary threads write it.  Tile bases must be 1024-byte aligned.
//   K-major operand  : row = M/N index, the 128 bytes hold 64 consecutive K elements;
//                      SBO = 1024 (next 8 rows), K advances by 32 bytes per MMA (K = 16).
//   MN-major operand : row = K index, the 128 bytes hold 64 consecutive M/N elements;
//                      SBO = 1024 (next 8 K), LBO = distance to the next 64 M/N elements,
//                      K advances by 2048 bytes per MMA.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace flab {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^31 clock ticks (about a second) and returns false, so a wrong
// descriptor or a lost arrival ends in an error code instead of a hung GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > (1ll << 31)) return false;
  }
}

// The same wait with a caller-chosen limit in clock ticks (the wait self-test uses a short one).
__device__ __forceinline__ bool mbar_wait_limit(uint64_t *bar, uint32_t parity, long long limit_ticks) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > limit_ticks) return false;
  }
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tile stores (shared -> global through a tensor map), tracked by the issuing thread's bulk groups. The writers
// of the shared tile execute fence_proxy_async() and synchronise with the issuing thread first.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(src)), "r"(c0),
               "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, const void *src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(smem_u32(src)),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the shared-memory sources of all of this thread's committed stores have been read
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// the same, but the most recently committed group may still be pending
__device__ __forceinline__ void tma_store_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// until all of this thread's committed stores are complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM ----------------------------------------------------------------------------------------
// Called by one full warp; writes the base address (lane 0, first column) to *dst in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t *dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ---------------------------------------------------------------------------------
// 64-bit shared-memory matrix descriptor, 128-byte swizzle, Blackwell descriptor version.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version 1
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// 32-bit instruction descriptor for kind::f16 with fp32 accumulation.
// ab_fmt: 0 = f16, 1 = bf16.  a_mn / b_mn: 1 = the operand is MN-major ("transposed").
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int ab_fmt, int a_mn, int b_mn) {
  return (1u << 4) | ((uint32_t)ab_fmt << 7) | ((uint32_t)ab_fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- MMA -----------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Makes `bar` complete once all MMAs issued so far by this thread have finished (implies
// tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// K-major operand: `kbytes_per_box` bytes between 64-element K boxes; issues kdim/16 MMAs.
// MN-major operand: 2048 bytes per K step.  The helpers below build the per-step descriptors.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int kstep, uint32_t box_bytes) {
  // kstep counts 16-element K steps; 4 steps per 128-byte box
  return smem_desc(tile + (uint32_t)(kstep >> 2) * box_bytes + (uint32_t)(kstep & 3) * 32u, 16u, 1024u);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int kstep, uint32_t mn_box_bytes) {
  return smem_desc(tile + (uint32_t)kstep * 2048u, mn_box_bytes, 1024u);
}

// ---- TMEM loads: 16 lanes x (8 * X) fp32 columns into the mma.sync m16n8 accumulator fragment layout:
//      thread t: r[4j+0..1] = (lane t/4,   cols 8j + 2(t%4) + {0,1}),  r[4j+2..3] = (lane t/4 + 8, same cols)
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, float (&r)[32]) {
  uint32_t *u = reinterpret_cast<uint32_t *>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, float (&r)[16]) {
  uint32_t *u = reinterpret_cast<uint32_t *>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 32 fp32 columns: thread t of the warp gets lane (quadrant base + t), r[j] = column j
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, float (&r)[32]) {
  uint32_t *u = reinterpret_cast<uint32_t *>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, float (&r)[8]) {
  uint32_t *u = reinterpret_cast<uint32_t *>(r);
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Load a [16 x 8*NI] block (NI multiple of 4) into acc[NI][4]; taddr = lane/column of its corner.
template <int NI> __device__ __forceinline__ void tmem_ld_frag(uint32_t taddr, float (&acc)[NI][4]) {
  static_assert(NI % 4 == 0 || NI == 2, "NI must be 2 or a multiple of 4");
  if constexpr (NI == 2) {
    float(&blk)[8] = *reinterpret_cast<float(*)[8]>(&acc[0][0]);
    tmem_ld_16x256b_x2(taddr, blk);
  } else {
#pragma unroll
    for (int j = 0; j < NI / 8; ++j) {
      float(&blk)[32] = *reinterpret_cast<float(*)[32]>(&acc[8 * j][0]);
      tmem_ld_16x256b_x8(taddr + 64u * j, blk);
    }
    if constexpr (NI % 8 != 0) {
      float(&blk)[16] = *reinterpret_cast<float(*)[16]>(&acc[NI - 4][0]);
      tmem_ld_16x256b_x4(taddr + 8u * (NI - 4), blk);
    }
  }
}

// ---- swizzled shared-memory addressing for ordinary threads ---------------------------------------
// byte offset of bf16 element (row, col) inside a [rows][64] 128-byte-swizzled tile
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  return (uint32_t)row * 128u + ((((uint32_t)col >> 3) ^ ((uint32_t)row & 7u)) << 4) + (((uint32_t)col & 7u) << 1);
}

// barrier among a subset of the CTA's warps (id 1..15, nthreads multiple of 32)
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Each translation unit with tcgen05 kernels defines its own device error word with this macro; a
// kernel whose bounded wait ran out stores an id of the wait there, and flab_tc_error_state() reads
// every unit's word through the generated host getter; getter##_clear() zeroes the word again.
#define FLAB_TC_DEFINE_ERROR_WORD(getter)                                            \
  namespace {                                                                        \
  __device__ int tu_tc_error = 0;                                                    \
  }                                                                                  \
  namespace flab {                                                                   \
  int getter() {                                                                     \
    int v = 0;                                                                       \
    if (cudaMemcpyFromSymbol(&v, tu_tc_error, sizeof(int)) != cudaSuccess) return -1000; \
    return v;                                                                        \
  }                                                                                  \
  int getter##_clear() {                                                             \
    const int v = 0;                                                                 \
    return cudaMemcpyToSymbol(tu_tc_error, &v, sizeof(int)) == cudaSuccess ? 0 : -1000; \
  }                                                                                  \
  }

}  // namespace tc

// Tensor map over a token-major tensor with inner extent D (multiple of 64): 4-D, 64-column boxes of
// 64 tokens.  seq-first [B,T,H,D]: dims (D, H, T, B), coordinates (d, h, t, b);
// head-first [B,H,T,D]: dims (D, T, H, B), coordinates (d, t, h, b).  Rows past T are zero-filled.
int make_token_map(CUtensorMap *map, const void *base, const flab_args *a, int D);
// Tensor map over chunk states [rows = NT*H*K][V], boxes of 64 columns x `box_rows` rows.
int make_state_map(CUtensorMap *map, const void *base, const flab_args *a, int box_rows);

// host: tensor-map construction without linking libcuda (entry point fetched from the runtime)
int make_tensor_map_bf16(CUtensorMap *map, const void *base, int rank, const uint64_t *dims, const uint64_t *strides_bytes,
                         const uint32_t *box, int elem_fp16);

}  // namespace flab
