// Self-check of the tcgen05 / TMEM / TMA plumbing: four small products that exercise every operand
// form the kernels use (K-major and MN-major A and B, M = 64 and M = 128, thread-written swizzled
// operand), read back with the fragment loads.  Single CTA; every wait is bounded.
#include "tc.cuh"

FLAB_TC_DEFINE_ERROR_WORD(tc_selftest_error)

namespace flab {

// A wait that is meant to run out: one warp waits, with a caller-chosen short limit, on an mbarrier that nothing
// ever arrives at.  It takes the same way out as a production kernel whose wait gave up: the id of the wait goes
// to the unit's error word (and to *status), the kernel returns normally and the context stays usable.
constexpr int WAIT_SELFTEST_ID = 99;
__global__ void __launch_bounds__(32) tc_wait_selftest_kernel(long long limit_ticks, int *status) {
  using namespace tc;
  __shared__ uint64_t never;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    fence_barrier_init();
  }
  __syncwarp();
  const bool ok = mbar_wait_limit(&never, 0, limit_ticks);
  if (threadIdx.x == 0) {
    if (!ok) atomicCAS(&tu_tc_error, 0, WAIT_SELFTEST_ID);
    *status = ok ? 0 : WAIT_SELFTEST_ID;
  }
}

__global__ void __launch_bounds__(128) tc_selftest_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                          const __grid_constant__ CUtensorMap mapH, const __grid_constant__ CUtensorMap mapV,
                                                          float *out, int *status) {
  using namespace tc;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve 1024-byte aligned tiles
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sA = base;            // [2 boxes][64][128B]   16 KB
  unsigned char *sB = sA + 16384;      // [2][64][128B]         16 KB
  unsigned char *sH = sB + 16384;      // [2][128][128B]        32 KB
  unsigned char *sV = sH + 32768;      // [64][128B]             8 KB
  unsigned char *sP = sV + 8192;       // [64][128B]             8 KB
  __shared__ uint64_t bar_tma, bar_mma[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&bar_tma, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_mma[i], 1);
    fail = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  if (tid == 0) {
    mbar_expect_tx(&bar_tma, 16384 + 16384 + 32768 + 8192);
    tma_load_2d(sA, &mapA, &bar_tma, 0, 0);
    tma_load_2d(sA + 8192, &mapA, &bar_tma, 64, 0);
    tma_load_2d(sB, &mapB, &bar_tma, 0, 0);
    tma_load_2d(sB + 8192, &mapB, &bar_tma, 64, 0);
    tma_load_2d(sH, &mapH, &bar_tma, 0, 0);
    tma_load_2d(sH + 16384, &mapH, &bar_tma, 64, 0);
    tma_load_2d(sV, &mapV, &bar_tma, 0, 0);
  }
  if (!mbar_wait(&bar_tma, 0)) atomicExch(&fail, 1);
  __syncthreads();
  if (fail == 0 && tid == 0) {
    fence_after_sync();
    const uint32_t a = smem_u32(sA), b = smem_u32(sB), h = smem_u32(sH), v = smem_u32(sV);
    // D1[64x64] = A B^T : both K-major, K = 128
    constexpr uint32_t i1 = instr_desc(64, 64, 1, 0, 0);
    for (int s = 0; s < 8; ++s) umma(tmem + 0, desc_kmajor(a, s, 8192), desc_kmajor(b, s, 8192), i1, s > 0);
    umma_commit(&bar_mma[0]);
    // D2[64x128] = A H : A K-major, B MN-major (two 64-column boxes of 128 rows, 16 KB apart)
    constexpr uint32_t i2 = instr_desc(64, 128, 1, 0, 1);
    for (int s = 0; s < 8; ++s) umma(tmem + 64, desc_kmajor(a, s, 8192), desc_mnmajor(h, s, 16384), i2, s > 0);
    umma_commit(&bar_mma[1]);
    // D3[128x64] = A^T V : A MN-major (M = 128 channels in two boxes 8 KB apart, K = 64 tokens), B MN-major
    constexpr uint32_t i3 = instr_desc(128, 64, 1, 1, 1);
    for (int s = 0; s < 4; ++s) umma(tmem + 192, desc_mnmajor(a, s, 8192), desc_mnmajor(v, s, 8192), i3, s > 0);
    umma_commit(&bar_mma[2]);
  }
  // D1 -> out, and P = bf16(D1) as a thread-written swizzled K-major operand
  float acc[8][4];
  if (fail == 0 && !mbar_wait(&bar_mma[0], 0)) atomicExch(&fail, 2);
  __syncthreads();
  if (fail == 0) {
    fence_after_sync();
    tmem_ld_frag<8>(tmem + ((uint32_t)(32 * warp) << 16) + 0, acc);
    tmem_ld_wait();
    const int g = lane >> 2, t4 = lane & 3;
    for (int ni = 0; ni < 8; ++ni)
      for (int r = 0; r < 4; ++r) {
        int row = 16 * warp + g + ((r >> 1) << 3), col = 8 * ni + 2 * t4 + (r & 1);
        out[row * 64 + col] = acc[ni][r];
        *reinterpret_cast<bf16 *>(sP + sw128_offset(row, col)) = __float2bfloat16_rn(acc[ni][r]);
      }
    fence_proxy_async();
  }
  fence_before_sync();
  __syncthreads();
  if (fail == 0 && tid == 0) {
    fence_after_sync();
    // D4[64x64] = P V : A K-major (K = 64), B MN-major
    constexpr uint32_t i4 = instr_desc(64, 64, 1, 0, 1);
    for (int s = 0; s < 4; ++s) umma(tmem + 256, desc_kmajor(smem_u32(sP), s, 8192), desc_mnmajor(smem_u32(sV), s, 8192), i4, s > 0);
    umma_commit(&bar_mma[3]);
  }
  float *out2 = out + 64 * 64, *out3 = out2 + 64 * 128, *out4 = out3 + 128 * 64;
  if (fail == 0 && !mbar_wait(&bar_mma[1], 0)) atomicExch(&fail, 3);
  if (fail == 0 && !mbar_wait(&bar_mma[2], 0)) atomicExch(&fail, 4);
  if (fail == 0 && !mbar_wait(&bar_mma[3], 0)) atomicExch(&fail, 5);
  __syncthreads();
  if (fail == 0) {
    fence_after_sync();
    const int g = lane >> 2, t4 = lane & 3;
    float acc2[16][4];
    tmem_ld_frag<16>(tmem + ((uint32_t)(32 * warp) << 16) + 64, acc2);
    tmem_ld_wait();
    for (int ni = 0; ni < 16; ++ni)
      for (int r = 0; r < 4; ++r) out2[(16 * warp + g + ((r >> 1) << 3)) * 128 + 8 * ni + 2 * t4 + (r & 1)] = acc2[ni][r];
    for (int half = 0; half < 2; ++half) {  // M = 128: lane = row
      tmem_ld_frag<8>(tmem + ((uint32_t)(32 * warp + 16 * half) << 16) + 192, acc);
      tmem_ld_wait();
      for (int ni = 0; ni < 8; ++ni)
        for (int r = 0; r < 4; ++r) out3[(32 * warp + 16 * half + g + ((r >> 1) << 3)) * 64 + 8 * ni + 2 * t4 + (r & 1)] = acc[ni][r];
    }
    tmem_ld_frag<8>(tmem + ((uint32_t)(32 * warp) << 16) + 256, acc);
    tmem_ld_wait();
    for (int ni = 0; ni < 8; ++ni)
      for (int r = 0; r < 4; ++r) out4[(16 * warp + g + ((r >> 1) << 3)) * 64 + 8 * ni + 2 * t4 + (r & 1)] = acc[ni][r];
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0) *status = fail;
}

}  // namespace flab

extern "C" int flab_tc_wait_selftest(long long limit_ticks, int *status, void *stream) {
  using namespace flab;
  FLAB_REQUIRE(status != nullptr, FLAB_E_BADARG, "tc_wait_selftest: NULL status");
  FLAB_REQUIRE(limit_ticks > 0 && limit_ticks <= (1ll << 28), FLAB_E_BADARG,
               "tc_wait_selftest: the limit must be between 1 and 2^28 clock ticks (a fraction of a second)");
  tc_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_ticks, status);
  return check_launch("tc_wait_selftest");
}

extern "C" int flab_tc_selftest(const void *a, const void *b, const void *h, const void *v, float *out, int *status, void *stream) {
  using namespace flab;
  FLAB_REQUIRE(a && b && h && v && out && status, FLAB_E_BADARG, "tc_selftest: NULL argument");
  CUtensorMap mA, mB, mH, mV;
  const uint64_t d_ab[2] = {128, 64}, s_ab[1] = {256};
  const uint32_t box_ab[2] = {64, 64};
  const uint64_t d_h[2] = {128, 128}, s_h[1] = {256};
  const uint32_t box_h[2] = {64, 128};
  const uint64_t d_v[2] = {64, 64}, s_v[1] = {128};
  const uint32_t box_v[2] = {64, 64};
  if (int e = make_tensor_map_bf16(&mA, a, 2, d_ab, s_ab, box_ab, 0)) return e;
  if (int e = make_tensor_map_bf16(&mB, b, 2, d_ab, s_ab, box_ab, 0)) return e;
  if (int e = make_tensor_map_bf16(&mH, h, 2, d_h, s_h, box_h, 0)) return e;
  if (int e = make_tensor_map_bf16(&mV, v, 2, d_v, s_v, box_v, 0)) return e;
  const size_t smem = 16384 + 16384 + 32768 + 8192 + 8192 + 1024;
  if (int e = set_smem(tc_selftest_kernel, smem)) return e;
  tc_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(mA, mB, mH, mV, out, status);
  return check_launch("tc_selftest");
}
