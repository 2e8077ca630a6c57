// 64x64 unit-lower-triangular inverse used by the WY kernels (fla/ops/delta_rule/wy_fast.py:94-253 computes the
// same matrix with a 16x16 forward substitution and fp32 block merges).
#pragma once
#include "common.cuh"

namespace flab {

constexpr int LDL = C + 1;  // leading dimension of the fp32 work matrices

template <int BAR> __device__ __forceinline__ void inverse_sync() {
  if (BAR == 0) __syncthreads();
  else asm volatile("bar.sync %0, 256;" ::"n"(BAR) : "memory");
}

// fp32 tile product on the tensor cores with a three-term bf16 split: x = hi + lo (both bf16), and
// x y ~= hi_x hi_y + hi_x lo_y + lo_x hi_y with fp32 accumulation. The relative error, about 2^-16, is two
// orders of magnitude below the rounding of the inverse to a 16-bit element type that follows, and the block
// merges drop from hundreds of shared-memory loads and FMAs per thread to a handful of MMAs.
// Same operand and accumulator conventions as warp_gemm_f32<1, NI, KD, false, true> (A row-major, B[k][n]).
template <int NI, int KD>
__device__ __forceinline__ void warp_mma_f32split(float (&acc)[1][NI][4], const float *A, int lda, int m0, const float *B, int ldb,
                                                  int n0) {
  static_assert(KD % 16 == 0, "contraction length must be a multiple of 16");
  const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  auto split = [](float x0, float x1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
  };
#pragma unroll
  for (int k0 = 0; k0 < KD; k0 += 16) {
    uint32_t ah[4], al[4];
    const float *a_lo = A + (m0 + g) * lda + k0 + 2 * t4, *a_hi = a_lo + 8 * lda;
    split(a_lo[0], a_lo[1], ah[0], al[0]);
    split(a_hi[0], a_hi[1], ah[1], al[1]);
    split(a_lo[8], a_lo[9], ah[2], al[2]);
    split(a_hi[8], a_hi[9], ah[3], al[3]);
#pragma unroll
    for (int ni = 0; ni < NI; ++ni) {
      const float *b = B + (k0 + 2 * t4) * ldb + n0 + ni * 8 + g;
      uint32_t bh0, bl0, bh1, bl1;
      split(b[0], b[ldb], bh0, bl0);
      split(b[8 * ldb], b[9 * ldb], bh1, bl1);
      mma16816<bf16>(acc[0][ni], al, bh0, bh1);
      mma16816<bf16>(acc[0][ni], ah, bl0, bl1);
      mma16816<bf16>(acc[0][ni], ah, bh0, bh1);
    }
  }
}

// In-place variant for 256 threads: X holds NMAT negated strict-lower Gram matrices ([64][LDL] fp32 each, zero
// on and above the diagonal) and leaves their inverses (unit diagonal included). Same blocked scheme as
// tri_inverse; every level reads a block into registers or scratch before it is overwritten. Scr is scratch of
// NMAT * 32 * 33 floats. All 256 threads must call this; BAR = 0 synchronises them with __syncthreads(), BAR > 0
// with the named barrier of that id (a 256-thread group inside a larger CTA; tid is then the index in the group).
template <int NMAT, int BAR = 0> __device__ __forceinline__ void tri_inverse8(float *X, float *Scr, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  // ---- level 0: warps 0..3 -> diagonal block, half-warp -> matrix
  if (warp < 4) {
    const int half = lane >> 4, j = lane & 15, mat = half < NMAT ? half : 0;
    float *n = X + mat * C * LDL + (16 * warp) * (LDL + 1);
    float nc[16], x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) nc[i] = n[i * LDL + j];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float acc = nc[i];
#pragma unroll
      for (int m = 0; m < i; ++m) acc = fmaf(__shfl_sync(0xffffffffu, nc[i], (lane & 16) + m), x[m], acc);
      x[i] = (j < i) ? acc : 0.f;
    }
    __syncwarp();
    if (half < NMAT) {
#pragma unroll
      for (int i = 0; i < 16; ++i) n[i * LDL + j] = x[i] + (i == j ? 1.f : 0.f);
    }
  }
  inverse_sync<BAR>();
  // ---- level 1: X21 = X22 (N21 X11); warp -> (matrix, 32-block, 8-column half of the 16x16 result)
  {
    const int mat = (warp >> 1) & 1, blk = warp & 1, n0 = 8 * (warp >> 2);
    const bool on = mat < NMAT;
    const int o = 32 * blk;
    float *Xm = X + (on ? mat : 0) * C * LDL;
    float *scr = Scr + ((on ? mat : 0) * 2 + blk) * 16 * 17;
    if (on) {
      float t1[1][1][4];
      acc_zero(t1);
      warp_mma_f32split<1, 16>(t1, Xm + (o + 16) * LDL + o, LDL, 0, Xm + o * LDL + o, LDL, n0);
      FLAB_ACC_FOREACH(1, 1, 0, n0, row, col, mi, ni, r) { scr[row * 17 + col] = t1[mi][ni][r]; }
    }
    inverse_sync<BAR>();
    if (on) {
      float t2[1][1][4];
      acc_zero(t2);
      warp_mma_f32split<1, 16>(t2, Xm + (o + 16) * LDL + o + 16, LDL, 0, scr, 17, n0);
      FLAB_ACC_FOREACH(1, 1, 0, n0, row, col, mi, ni, r) { Xm[(o + 16 + row) * LDL + o + col] = t2[mi][ni][r]; }
    }
  }
  inverse_sync<BAR>();
  // ---- level 2: X_BA = X_BB (N_BA X_AA); two matrices: warp -> (matrix, 16x16 tile); one: warp -> 16x8 tile
  {
    constexpr int NI2 = NMAT == 2 ? 2 : 1;
    const int mat = NMAT == 2 ? (warp >> 2) : 0, tile = NMAT == 2 ? (warp & 3) : warp;
    const int m0 = 16 * (tile & 1), n0 = 8 * NI2 * (tile >> 1);
    float *Xm = X + mat * C * LDL;
    float *scr = Scr + mat * 32 * 33;
    float t1[1][NI2][4];
    acc_zero(t1);
    warp_mma_f32split<NI2, 32>(t1, Xm + 32 * LDL, LDL, m0, Xm, LDL, n0);
    FLAB_ACC_FOREACH(1, NI2, m0, n0, row, col, mi, ni, r) { scr[row * 33 + col] = t1[mi][ni][r]; }
    inverse_sync<BAR>();
    float t2[1][NI2][4];
    acc_zero(t2);
    warp_mma_f32split<NI2, 32>(t2, Xm + 32 * LDL + 32, LDL, m0, scr, 33, n0);
    FLAB_ACC_FOREACH(1, NI2, m0, n0, row, col, mi, ni, r) { Xm[(32 + row) * LDL + col] = t2[mi][ni][r]; }
  }
  inverse_sync<BAR>();
}

}  // namespace flab
