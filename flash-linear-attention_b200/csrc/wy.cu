// WY / UT transform of the (gated) delta rule, one CTA per (chunk, head).
//   forward : A = (I + tril(diag(beta) K K^T [* e^{b_i-b_j}], -1))^-1,  w = Aw (beta k),  u = Au (beta v)
//             (fla/ops/delta_rule/wy_fast.py:94-253, fla/ops/gated_delta_rule/wy_fast.py:111-317)
//   backward: dk, dv, dbeta (, dg) from dw, du through the inverse
//             (fla/ops/delta_rule/wy_fast.py:325-433, fla/ops/gated_delta_rule/wy_fast.py:440-562)
// The Gram matrix and all products run on the tensor cores; the 64x64 unit-lower-triangular inverse
// is a forward substitution in fp32 shared memory (one thread per column, one barrier per row).
// A is rounded to the element type before it multiplies anything, as in the reference.
// K and V are walked in tiles of 128 columns, so any head dimension works.
#include "common.cuh"
#include "wy_inverse.cuh"

namespace flab {

constexpr int WT = 128;  // column tile of k / v

// Inverse of the unit lower-triangular M = I - N for `nmat` 64x64 matrices held side by side in
// shared memory (N = Lo, the negated strict lower part of the Gram matrix).  Result X = M^-1
// (with its unit diagonal) is written to Xo.  Blocked scheme:
//   1. the four 16x16 diagonal blocks: forward substitution in registers, one half-warp per block
//      (lane = column, coefficients broadcast with shuffles);
//   2. 32x32 level:  X21 = X22 N21 X11 for both 32-blocks;
//   3. 64x64 level:  X_BA = X_BB N_BA X_AA.
// Levels 2 and 3 are small fp32 FFMA tile products (true fp32, like the reference's tl.dot with
// allow_tf32=False).  Scr is scratch of nmat * 32 * 33 floats.  All 128 threads must call this.
__device__ __forceinline__ void tri_inverse(const float *Lo, float *Xo, float *Scr, int nmat, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  // only the blocks above the block diagonal are read before they are written: zero those
  for (int e = tid; e < nmat * 32 * 32; e += 128) {
    const int m = e >> 10, r = (e >> 5) & 31, c = e & 31;
    Xo[m * C * LDL + r * LDL + 32 + c] = 0.f;                                  // rows 0..31, cols 32..63
    if ((r < 16) && (c >= 16)) {
      Xo[m * C * LDL + r * LDL + c] = 0.f;                                     // rows 0..15, cols 16..31
      Xo[m * C * LDL + (32 + r) * LDL + 32 + c] = 0.f;                         // rows 32..47, cols 48..63
    }
  }
  __syncthreads();
  // ---- level 0: 16x16 diagonal blocks; warp w -> diagonal block w, half-warp -> matrix
  {
    const int half = lane >> 4, j = lane & 15, mat = half < nmat ? half : 0;
    const float *n = Lo + mat * C * LDL + (16 * warp) * LDL + 16 * warp;
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
    if (half < nmat) {
      float *xo = Xo + mat * C * LDL + (16 * warp) * LDL + 16 * warp;
#pragma unroll
      for (int i = 0; i < 16; ++i) xo[i * LDL + j] = x[i] + (i == j ? 1.f : 0.f);
    }
  }
  __syncthreads();
  // ---- level 1: warp -> (matrix, 32-block); X21 = X22 (N21 X11)
  {
    const int mat = warp >> 1, blk = warp & 1;
    if (mat < nmat) {
      const int o = 32 * blk;
      const float *N21 = Lo + mat * C * LDL + (o + 16) * LDL + o;
      float *X = Xo + mat * C * LDL;
      float *scr = Scr + warp * 16 * 17;
      float t1[1][2][4];
      acc_zero(t1);
      warp_gemm_f32<1, 2, 16, false, true>(t1, N21, LDL, 0, X + o * LDL + o, LDL, 0);
      FLAB_ACC_FOREACH(1, 2, 0, 0, row, col, mi, ni, r) { scr[row * 17 + col] = t1[mi][ni][r]; }
      __syncwarp();
      float t2[1][2][4];
      acc_zero(t2);
      warp_gemm_f32<1, 2, 16, false, true>(t2, X + (o + 16) * LDL + o + 16, LDL, 0, scr, 17, 0);
      __syncwarp();
      FLAB_ACC_FOREACH(1, 2, 0, 0, row, col, mi, ni, r) { X[(o + 16 + row) * LDL + o + col] = t2[mi][ni][r]; }
    }
  }
  __syncthreads();
  // ---- level 2: X_BA = X_BB (N_BA X_AA); warp -> 16x16 tile of the 32x32 result, per matrix
  {
    const int m0 = 16 * (warp & 1), n0 = 16 * (warp >> 1);
    for (int mat = 0; mat < nmat; ++mat) {
      const float *N = Lo + mat * C * LDL + 32 * LDL;  // rows 32.., cols 0..
      const float *X = Xo + mat * C * LDL;
      float t1[1][2][4];
      acc_zero(t1);
      warp_gemm_f32<1, 2, 32, false, true>(t1, N, LDL, m0, X, LDL, n0);
      FLAB_ACC_FOREACH(1, 2, m0, n0, row, col, mi, ni, r) { Scr[mat * 32 * 33 + row * 33 + col] = t1[mi][ni][r]; }
    }
    __syncthreads();
    for (int mat = 0; mat < nmat; ++mat) {
      float *X = Xo + mat * C * LDL;
      float t2[1][2][4];
      acc_zero(t2);
      warp_gemm_f32<1, 2, 32, false, true>(t2, X + 32 * LDL + 32, LDL, m0, Scr + mat * 32 * 33, 33, n0);
      FLAB_ACC_FOREACH(1, 2, m0, n0, row, col, mi, ni, r) { X[(32 + row) * LDL + col] = t2[mi][ni][r]; }
    }
  }
  __syncthreads();
}

template <typename T, bool GATED, bool RECOMPUTE>
__global__ void __launch_bounds__(128) wy_fwd_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LDX = WT + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  constexpr int NM = GATED ? 2 : 1;
  T *sX = reinterpret_cast<T *>(smem_raw);  // [64][LDX] k or v tile; reused to stage w / u
  T *sXB = sX + C * LDX;                    // [64][LDX] beta-scaled tile
  T *sA = sXB + C * LDX;                    // [NM][64][LDP] Aw, Au as T
  float *sBeta = reinterpret_cast<float *>(sA + NM * C * LDP);  // [64]
  float *sG = sBeta + C;                                        // [64]
  float *sLi = sG + C;                                          // [NM][64][LDL] inverse (not for RECOMPUTE)
  float *sScr = sLi + NM * C * LDL;                             // [NM][32][33] scratch of the inverse
  // the negated Gram matrices live in the (by then idle) k tile buffers while they are inverted
  float *sLo = reinterpret_cast<float *>(smem_raw);             // [NM][64][LDL]
  static_assert(2 * C * LDX * sizeof(T) >= (size_t)NM * C * LDL * sizeof(float), "Gram alias does not fit");

  const int tid = threadIdx.x, warp = tid >> 5;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V), offa = tok_off(a, s, hd, t0, C);
  const T *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v), *beta = reinterpret_cast<const T *>(a.beta);
  const int m0 = warp * 16;

  if (tid < C) {
    sBeta[tid] = tid < rows ? Num<T>::f(beta[tok_off(a, s, hd, t0 + tid, 1)]) : 0.f;
    // the gate only enters through the Gram decay, which the recompute path does not rebuild
    sG[tid] = (GATED && !RECOMPUTE && tid < rows) ? reinterpret_cast<const float *>(a.g)[tok_off(a, s, hd, t0 + tid, 1)] : 0.f;
  }

  if (!RECOMPUTE) {
    float gram[1][8][4];
    acc_zero(gram);
    for (int k0 = 0; k0 < a.K; k0 += WT) {
      const int kw = min(WT, a.K - k0), kp = round_up(kw, 16);
      __syncthreads();
      tile_load<T>(sX, LDX, k + offk + k0, ks, rows, C, kw, kp, tid, 128);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      tile_scale_rows<T>(sXB, sX, LDX, kp, sBeta, tid, 128);
      __syncthreads();
      WarpGemm<1, 8, false, false, T>::run(gram, sXB, LDX, m0, sX, LDX, 0, kp);
    }
    __syncthreads();  // every warp is done reading the k tiles before the Gram matrices overwrite them
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) {
      float x = row > col ? -gram[mi][ni][r] : 0.f;
      sLo[row * LDL + col] = x;
      if (GATED) sLo[C * LDL + row * LDL + col] = row > col ? x * safe_fexp<T>(sG[row] - sG[col]) : 0.f;
    }
    __syncthreads();
    tri_inverse(sLo, sLi, sScr, NM, tid);
    for (int e = tid; e < NM * C * 8; e += 128) {  // 8 elements (16 bytes of T) per step
      const int m = e >> 9, r_ = (e >> 3) & 63, c_ = (e & 7) * 8;
      const float *src = sLi + m * C * LDL + r_ * LDL + c_;
      int4 x;
      T *px = reinterpret_cast<T *>(&x);
#pragma unroll
      for (int j = 0; j < 8; ++j) px[j] = Num<T>::t(src[j]);
      *reinterpret_cast<int4 *>(sA + m * C * LDP + r_ * LDP + c_) = x;
    }
    __syncthreads();
    tile_store<T>(reinterpret_cast<T *>(a.aw) + offa, as_, sA, LDP, rows, C, tid, 128);
    if (GATED) tile_store<T>(reinterpret_cast<T *>(a.au) + offa, as_, sA + C * LDP, LDP, rows, C, tid, 128);
  } else {
    tile_load<T>(sA, LDP, reinterpret_cast<const T *>(a.aw) + offa, as_, rows, C, C, C, tid, 128);
    if (GATED) tile_load<T>(sA + C * LDP, LDP, reinterpret_cast<const T *>(a.au) + offa, as_, rows, C, C, C, tid, 128);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
  }

  // w = Aw (beta k), u = Au (beta v), tile by tile
  for (int pass = 0; pass < 2; ++pass) {
    const int D = pass == 0 ? a.K : a.V;
    const T *src = pass == 0 ? k + offk : v + offv;
    T *dst = pass == 0 ? reinterpret_cast<T *>(a.w) + offk : reinterpret_cast<T *>(a.u) + offv;
    const size_t st = pass == 0 ? ks : vs;
    const T *A = (pass == 1 && GATED) ? sA + C * LDP : sA;
    for (int d0 = 0; d0 < D; d0 += WT) {
      const int dw_ = min(WT, D - d0);
      __syncthreads();
      tile_load<T>(sXB, LDX, src + d0, st, rows, C, dw_, WT, tid, 128);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      tile_scale_rows<T>(sXB, sXB, LDX, WT, sBeta, tid, 128);
      __syncthreads();
      float acc[1][16][4];
      acc_zero(acc);
      WarpGemm<1, 16, false, true, T>::run(acc, A, LDP, m0, sXB, LDX, 0, C);
      acc_to_smem<1, 16, T>(acc, sX, LDX, m0, 0);
      __syncthreads();
      tile_store<T>(dst + d0, st, sX, LDX, rows, dw_, tid, 128);
    }
  }
}

// Forward for 16-bit element types with K, V <= 128: eight warps, the whole k and v tiles of the chunk resident
// in shared memory (loaded once, v while the Gram matrix is built and inverted), three CTAs per SM.
//   * beta enters the Gram matrix as a row factor of the fp32 product and enters w, u as a COLUMN factor of A
//     (A diag(beta)) x = A (beta x), so no beta-scaled copy of k or v is made;
//   * the gated Gram matrix is the similarity transform D N D^-1 of the ungated one (D = diag(e^b)), hence
//     Au = D Aw D^-1, i.e. Au_ij = Aw_ij e^{b_i - b_j}: ONE inverse serves both;
//   * the scaled copies are derived from the rounded A, so the recompute entry (which reads the stored A)
//     produces bit-identical w and u.
template <typename T, bool GATED, bool RECOMPUTE>
__global__ void __launch_bounds__(256, 3) wy_fwd16_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LDX = WT + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  constexpr int NM = GATED ? 2 : 1;
  T *sK = reinterpret_cast<T *>(smem_raw);  // [64][LDX] k, replaced in place by w
  T *sV = sK + C * LDX;                     // [64][LDX] v, replaced in place by u
  T *sAb = sV + C * LDX;                    // [NM][64][LDP] Aw diag(beta), Au diag(beta)
  float *sBeta = reinterpret_cast<float *>(sAb + NM * C * LDP);  // [64]
  float *sG = sBeta + C;                                         // [64]
  float *sF = sG + C;                                            // [64][LDL] negated Gram matrix, inverted in place
  float *sScr = reinterpret_cast<float *>(sAb);                  // scratch of the inverse (sAb still idle)
  static_assert((size_t)NM * C * LDP * sizeof(T) >= (size_t)32 * 33 * sizeof(float), "inverse scratch does not fit");

  const int tid = threadIdx.x, warp = tid >> 5;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V), offa = tok_off(a, s, hd, t0, C);
  const T *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v), *beta = reinterpret_cast<const T *>(a.beta);
  const int m0 = (warp & 3) * 16, nh = warp >> 2;

  tile_load<T>(sK, LDX, k + offk, ks, rows, C, a.K, WT, tid, 256);
  if (RECOMPUTE) {
    tile_load<T>(sAb, LDP, reinterpret_cast<const T *>(a.aw) + offa, as_, rows, C, C, C, tid, 256);
    if (GATED) tile_load<T>(sAb + C * LDP, LDP, reinterpret_cast<const T *>(a.au) + offa, as_, rows, C, C, C, tid, 256);
  }
  cp_async_commit();
  tile_load<T>(sV, LDX, v + offv, vs, rows, C, a.V, WT, tid, 256);
  cp_async_commit();
  if (tid < C) {
    sBeta[tid] = tid < rows ? Num<T>::f(beta[tok_off(a, s, hd, t0 + tid, 1)]) : 0.f;
    // the gate only enters through the decay of A, which the recompute path does not rebuild
    sG[tid] = (GATED && !RECOMPUTE && tid < rows) ? reinterpret_cast<const float *>(a.g)[tok_off(a, s, hd, t0 + tid, 1)] : 0.f;
  }
  cp_async_wait<1>();
  __syncthreads();  // k (and the stored A) have landed

  if (!RECOMPUTE) {
    float gram[1][4][4];
    acc_zero(gram);
    WarpGemm<1, 4, false, false, T>::run(gram, sK, LDX, m0, sK, LDX, nh * 32, round_up(a.K, 16));
    FLAB_ACC_FOREACH(1, 4, m0, nh * 32, row, col, mi, ni, r) {
      sF[row * LDL + col] = row > col ? -gram[mi][ni][r] * sBeta[row] : 0.f;
    }
    __syncthreads();
    tri_inverse8<1>(sF, sScr, tid);
  }
  // A (forward: rounded and written to global from registers) and A diag(beta), 8 elements per step
  for (int e = tid; e < C * 8; e += 256) {
    const int r_ = e >> 3, c_ = (e & 7) * 8;
#pragma unroll
    for (int m = 0; m < NM; ++m) {
      T *pab = sAb + m * C * LDP + r_ * LDP + c_;
      int4 x;
      T *px = reinterpret_cast<T *>(&x);
      if (!RECOMPUTE) {
        const float *src = sF + r_ * LDL + c_;
#pragma unroll
        for (int j = 0; j < 8; ++j) px[j] = Num<T>::t(m == 0 ? src[j] : src[j] * safe_fexp<T>(sG[r_] - sG[c_ + j]));
        if (r_ < rows) *reinterpret_cast<int4 *>(reinterpret_cast<T *>(m == 0 ? a.aw : a.au) + offa + (size_t)r_ * as_ + c_) = x;
      } else {
        x = *reinterpret_cast<const int4 *>(pab);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) px[j] = Num<T>::t(Num<T>::f(px[j]) * sBeta[c_ + j]);
      *reinterpret_cast<int4 *>(pab) = x;
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // A diag(beta) and v are in place
  // w = (Aw diag(beta)) k, then u = (Au diag(beta)) v; warp tile 16 rows x 64 columns, results replace k and v
  const bool do_w = nh * 64 < a.K, do_u = nh * 64 < a.V;
  float acc[1][8][4];
  acc_zero(acc);
  if (do_w) WarpGemm<1, 8, false, true, T>::run(acc, sAb, LDP, m0, sK, LDX, nh * 64, C);
  __syncthreads();  // every warp has read k
  if (do_w) acc_to_smem<1, 8, T>(acc, sK, LDX, m0, nh * 64);
  acc_zero(acc);
  if (do_u) WarpGemm<1, 8, false, true, T>::run(acc, GATED ? sAb + C * LDP : sAb, LDP, m0, sV, LDX, nh * 64, C);
  __syncthreads();  // every warp has read v; w is complete
  if (do_u) acc_to_smem<1, 8, T>(acc, sV, LDX, m0, nh * 64);
  tile_store<T>(reinterpret_cast<T *>(a.w) + offk, ks, sK, LDX, rows, a.K, tid, 256);
  __syncthreads();
  tile_store<T>(reinterpret_cast<T *>(a.u) + offv, vs, sV, LDX, rows, a.V, tid, 256);
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
template <typename T, bool GATED>
__global__ void __launch_bounds__(128) wy_bwd_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LDX = WT + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  T *sX = reinterpret_cast<T *>(smem_raw);  // [64][LDX] k / v tile
  T *sXB = sX + C * LDX;                    // [64][LDX] beta-scaled tile
  T *sD = sXB + C * LDX;                    // [64][LDX] dw / du tile; reused to stage outputs
  T *sAw = sD + C * LDX;                    // [64][LDP]
  T *sAu = sAw + C * LDP;                   // [64][LDP] (gated)
  T *sDA = sAu + (GATED ? C * LDP : 0);     // [64][LDP] staged dA
  T *sTmp = sDA + C * LDP;                  // [64][LDP] staged intermediate product
  float *sBeta = reinterpret_cast<float *>(sTmp + C * LDP);  // [64]
  float *sG = sBeta + C;                                     // [64]
  float *sDG = sG + C;                                       // [64]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V), offa = tok_off(a, s, hd, t0, C);
  const T *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v), *beta = reinterpret_cast<const T *>(a.beta);
  const int m0 = warp * 16;

  if (tid < C) {
    sBeta[tid] = tid < rows ? Num<T>::f(beta[tok_off(a, s, hd, t0 + tid, 1)]) : 0.f;
    sG[tid] = (GATED && tid < rows) ? reinterpret_cast<const float *>(a.g)[tok_off(a, s, hd, t0 + tid, 1)] : 0.f;
    sDG[tid] = 0.f;
  }
  tile_load<T>(sAw, LDP, reinterpret_cast<const T *>(a.aw) + offa, as_, rows, C, C, C, tid, 128);
  if (GATED) tile_load<T>(sAu, LDP, reinterpret_cast<const T *>(a.au) + offa, as_, rows, C, C, C, tid, 128);
  cp_async_commit();

  const float b_lo = 0.f;
  (void)b_lo;
  float dbeta_lo = 0.f, dbeta_hi = 0.f;  // rows m0+g8, m0+g8+8 (partial over this thread's columns)
  float dA[1][8][4], dA2[1][8][4];
  acc_zero(dA);
  acc_zero(dA2);

  // one pass over the column tiles of (x = k or v, dx = dw or du): accumulates dAcc += dx (beta x)^T,
  // writes dout = (A^T dx) * beta and adds sum(A^T dx * x) to dbeta.
  auto tile_pass = [&](const T *x, const T *dx, T *dout, size_t st, int D, const T *A, float (&dAcc)[1][8][4]) {
    for (int d0 = 0; d0 < D; d0 += WT) {
      const int dw_ = min(WT, D - d0);
      __syncthreads();
      tile_load<T>(sX, LDX, x + d0, st, rows, C, dw_, WT, tid, 128);
      tile_load<T>(sD, LDX, dx + d0, st, rows, C, dw_, WT, tid, 128);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      tile_scale_rows<T>(sXB, sX, LDX, WT, sBeta, tid, 128);
      __syncthreads();
      WarpGemm<1, 8, false, false, T>::run(dAcc, sD, LDX, m0, sXB, LDX, 0, WT);
      float acc[1][16][4];
      acc_zero(acc);
      WarpGemm<1, 16, true, true, T>::run(acc, A, LDP, m0, sD, LDX, 0, C);
      FLAB_ACC_FOREACH(1, 16, m0, 0, row, col, mi, ni, r) {
        float xb = acc[mi][ni][r];
        float xv = Num<T>::f(sX[row * LDX + col]);
        if (r >> 1) dbeta_hi += xb * xv; else dbeta_lo += xb * xv;
        acc[mi][ni][r] = xb * sBeta[row];
      }
      __syncthreads();  // all warps finished reading sD
      acc_to_smem<1, 16, T>(acc, sD, LDX, m0, 0);
      __syncthreads();
      tile_store<T>(dout + d0, st, sD, LDX, rows, dw_, tid, 128);
    }
  };
  // dA <- -strict_lower(A^T strict_lower(dA) A^T), rounded to T between products; result left in
  // registers (rounded) and staged in sDA.
  auto transform = [&](float (&dAcc)[1][8][4], const T *A) {
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) { dAcc[mi][ni][r] = row > col ? dAcc[mi][ni][r] : 0.f; }
    __syncthreads();
    acc_to_smem<1, 8, T>(dAcc, sDA, LDP, m0, 0);
    __syncwarp();
    float x1[1][8][4];
    acc_zero(x1);
    WarpGemm<1, 8, false, false, T>::run(x1, sDA, LDP, m0, A, LDP, 0, C);  // dA A^T
    acc_to_smem<1, 8, T>(x1, sTmp, LDP, m0, 0);
    __syncthreads();
    acc_zero(dAcc);
    WarpGemm<1, 8, true, true, T>::run(dAcc, A, LDP, m0, sTmp, LDP, 0, C);  // A^T (dA A^T)
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) { dAcc[mi][ni][r] = row > col ? rnd<T>(-dAcc[mi][ni][r]) : 0.f; }
  };

  cp_async_wait<0>();
  __syncthreads();
  T *dk = reinterpret_cast<T *>(a.dk) + offk, *dv = reinterpret_cast<T *>(a.dv) + offv;
  const T *dw = reinterpret_cast<const T *>(a.dw) + offk, *du = reinterpret_cast<const T *>(a.du) + offv;
  if (!GATED) {
    tile_pass(v + offv, du, dv, vs, a.V, sAw, dA);
    tile_pass(k + offk, dw, dk, ks, a.K, sAw, dA);
    transform(dA, sAw);
  } else {
    tile_pass(k + offk, dw, dk, ks, a.K, sAw, dA);
    transform(dA, sAw);
    tile_pass(v + offv, du, dv, vs, a.V, sAu, dA2);
    transform(dA2, sAu);
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) {
      float x2 = dA2[mi][ni][r] * safe_fexp<T>(sG[row] - sG[col]);
      dA2[mi][ni][r] = x2;
      dA[mi][ni][r] = rnd<T>(dA[mi][ni][r] + x2);
    }
  }
  __syncthreads();
  acc_to_smem<1, 8, T>(dA, sDA, LDP, m0, 0);
  __syncthreads();

  // second K pass: dk += dA^T (beta k) + (dA k) * beta; dbeta += sum((dA k) * k); gated: Gram for dg
  float gram[1][8][4];
  acc_zero(gram);
  for (int k0 = 0; k0 < a.K; k0 += WT) {
    const int kw = min(WT, a.K - k0);
    __syncthreads();
    tile_load<T>(sX, LDX, k + offk + k0, ks, rows, C, kw, WT, tid, 128);
    tile_load<T>(sD, LDX, dk + k0, ks, rows, C, kw, WT, tid, 128);  // first-pass dk (rounded to T)
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    tile_scale_rows<T>(sXB, sX, LDX, WT, sBeta, tid, 128);
    __syncthreads();
    if (GATED) WarpGemm<1, 8, false, false, T>::run(gram, sXB, LDX, m0, sX, LDX, 0, WT);
    float kb2[1][16][4], acc[1][16][4];
    acc_zero(kb2);
    acc_zero(acc);
    WarpGemm<1, 16, false, true, T>::run(kb2, sDA, LDP, m0, sX, LDX, 0, C);  // dA k
    WarpGemm<1, 16, true, true, T>::run(acc, sDA, LDP, m0, sXB, LDX, 0, C);  // dA^T (beta k)
    FLAB_ACC_FOREACH(1, 16, m0, 0, row, col, mi, ni, r) {
      float xb = kb2[mi][ni][r];
      float kv = Num<T>::f(sX[row * LDX + col]);
      if (r >> 1) dbeta_hi += xb * kv; else dbeta_lo += xb * kv;
      acc[mi][ni][r] += Num<T>::f(sD[row * LDX + col]) + xb * sBeta[row];
      if (a.x && row < rows && col < kw) acc[mi][ni][r] += Num<T>::f(reinterpret_cast<const T *>(a.x)[offk + (size_t)row * ks + k0 + col]);
    }
    // each thread overwrites exactly the sD elements it just read
    acc_to_smem<1, 16, T>(acc, sD, LDX, m0, 0);
    __syncthreads();
    tile_store<T>(dk + k0, ks, sD, LDX, rows, kw, tid, 128);
  }
  // dbeta
  dbeta_lo += __shfl_xor_sync(0xffffffffu, dbeta_lo, 1);
  dbeta_lo += __shfl_xor_sync(0xffffffffu, dbeta_lo, 2);
  dbeta_hi += __shfl_xor_sync(0xffffffffu, dbeta_hi, 1);
  dbeta_hi += __shfl_xor_sync(0xffffffffu, dbeta_hi, 2);
  float *dbeta = reinterpret_cast<float *>(a.dbeta);
  if ((lane & 3) == 0) {
    if (m0 + g8 < rows) dbeta[tok_off(a, s, hd, t0 + m0 + g8, 1)] = dbeta_lo;
    if (m0 + g8 + 8 < rows) dbeta[tok_off(a, s, hd, t0 + m0 + g8 + 8, 1)] = dbeta_hi;
  }
  if (GATED) {
    // dg = rowsum(dA2 * Gram) - colsum(dA2 * Gram)
    float r_lo = 0.f, r_hi = 0.f;
#pragma unroll
    for (int ni = 0; ni < 8; ++ni) {
      float p0 = dA2[0][ni][0] * gram[0][ni][0], p1 = dA2[0][ni][1] * gram[0][ni][1];
      float p2 = dA2[0][ni][2] * gram[0][ni][2], p3 = dA2[0][ni][3] * gram[0][ni][3];
      r_lo += p0 + p1;
      r_hi += p2 + p3;
      float c0 = p0 + p2, c1 = p1 + p3;
      c0 += __shfl_xor_sync(0xffffffffu, c0, 4);
      c0 += __shfl_xor_sync(0xffffffffu, c0, 8);
      c0 += __shfl_xor_sync(0xffffffffu, c0, 16);
      c1 += __shfl_xor_sync(0xffffffffu, c1, 4);
      c1 += __shfl_xor_sync(0xffffffffu, c1, 8);
      c1 += __shfl_xor_sync(0xffffffffu, c1, 16);
      if (g8 == 0) {
        atomicAdd(&sDG[ni * 8 + 2 * (lane & 3)], -c0);
        atomicAdd(&sDG[ni * 8 + 2 * (lane & 3) + 1], -c1);
      }
    }
    r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 1);
    r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 2);
    r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 1);
    r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 2);
    if ((lane & 3) == 0) {
      atomicAdd(&sDG[m0 + g8], r_lo);
      atomicAdd(&sDG[m0 + g8 + 8], r_hi);
    }
    __syncthreads();
    if (tid < rows) reinterpret_cast<float *>(a.dg)[tok_off(a, s, hd, t0 + tid, 1)] = sDG[tid];
  }
}

// Backward for 16-bit element types with K, V <= 128: eight warps; k, v, dw, du of the chunk are loaded once
// and stay resident (dk and dv are built in place over dw and du), two CTAs per SM. beta is applied to fp32
// accumulators (as a column factor of dw k^T, a row factor of k k^T) or to the 64x64 matrix dA instead of
// to a copy of k or v.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256, 2) wy_bwd16_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LDX = WT + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  T *sK = reinterpret_cast<T *>(smem_raw);  // [64][LDX] k
  T *sV = sK + C * LDX;                     // [64][LDX] v
  T *sDW = sV + C * LDX;                    // [64][LDX] dw, replaced in place by dk
  T *sDU = sDW + C * LDX;                   // [64][LDX] du, replaced in place by dv
  T *sAw = sDU + C * LDX;                   // [64][LDP]
  T *sAu = sAw + C * LDP;                   // [64][LDP] (gated)
  T *sDA = sAu + (GATED ? C * LDP : 0);     // [64][LDP] staged dA
  T *sTmp = sDA + C * LDP;                  // [64][LDP] staged intermediate product; later diag(beta) dA
  float *sBeta = reinterpret_cast<float *>(sTmp + C * LDP);  // [64]
  float *sG = sBeta + C;                                     // [64]
  float *sDG = sG + C;                                       // [64]
  float *sDB = sDG + C;                                      // [64]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V), offa = tok_off(a, s, hd, t0, C);
  const T *beta = reinterpret_cast<const T *>(a.beta);
  const int m0 = (warp & 3) * 16, n32 = (warp >> 2) * 32, n64 = (warp >> 2) * 64;

  tile_load<T>(sAw, LDP, reinterpret_cast<const T *>(a.aw) + offa, as_, rows, C, C, C, tid, 256);
  tile_load<T>(sK, LDX, reinterpret_cast<const T *>(a.k) + offk, ks, rows, C, a.K, WT, tid, 256);
  tile_load<T>(sDW, LDX, reinterpret_cast<const T *>(a.dw) + offk, ks, rows, C, a.K, WT, tid, 256);
  cp_async_commit();
  if (GATED) tile_load<T>(sAu, LDP, reinterpret_cast<const T *>(a.au) + offa, as_, rows, C, C, C, tid, 256);
  tile_load<T>(sV, LDX, reinterpret_cast<const T *>(a.v) + offv, vs, rows, C, a.V, WT, tid, 256);
  tile_load<T>(sDU, LDX, reinterpret_cast<const T *>(a.du) + offv, vs, rows, C, a.V, WT, tid, 256);
  cp_async_commit();
  if (tid < C) {
    sBeta[tid] = tid < rows ? Num<T>::f(beta[tok_off(a, s, hd, t0 + tid, 1)]) : 0.f;
    sG[tid] = (GATED && tid < rows) ? reinterpret_cast<const float *>(a.g)[tok_off(a, s, hd, t0 + tid, 1)] : 0.f;
    sDG[tid] = 0.f;
    sDB[tid] = 0.f;
  }

  float dbeta_lo = 0.f, dbeta_hi = 0.f;  // rows m0+g8, m0+g8+8 (partial over this thread's columns)
  float dA[1][4][4], dA2[1][4][4];
  acc_zero(dA);
  acc_zero(dA2);

  // one pass over (x = k or v, dx = dw or du): dAcc += dx x^T (beta is applied by `transform`), dx is replaced
  // in place by (A^T dx) * beta and sum(A^T dx * x) is added to dbeta.
  auto pass = [&](const T *sX, T *sDX, const T *A, int D, float (&dAcc)[1][4][4]) {
    WarpGemm<1, 4, false, false, T>::run(dAcc, sDX, LDX, m0, sX, LDX, n32, round_up(D, 16));
    const bool on = n64 < D;
    float acc[1][8][4];
    acc_zero(acc);
    if (on) {
      WarpGemm<1, 8, true, true, T>::run(acc, A, LDP, m0, sDX, LDX, n64, C);
      const float b_lo = sBeta[m0 + g8], b_hi = sBeta[m0 + g8 + 8];
#pragma unroll
      for (int ni = 0; ni < 8; ++ni) {
        const int col = n64 + ni * 8 + 2 * t4;
        const float2 x_lo = ld_pair<T>(sX + (m0 + g8) * LDX + col), x_hi = ld_pair<T>(sX + (m0 + g8 + 8) * LDX + col);
        dbeta_lo += acc[0][ni][0] * x_lo.x + acc[0][ni][1] * x_lo.y;
        dbeta_hi += acc[0][ni][2] * x_hi.x + acc[0][ni][3] * x_hi.y;
        acc[0][ni][0] *= b_lo;
        acc[0][ni][1] *= b_lo;
        acc[0][ni][2] *= b_hi;
        acc[0][ni][3] *= b_hi;
      }
    }
    __syncthreads();  // every warp has read dx
    if (on) acc_to_smem<1, 8, T>(acc, sDX, LDX, m0, n64);
  };
  // dAcc <- -strict_lower(A^T strict_lower(dAcc diag(beta)) A^T), rounded to T between products; the result
  // stays in registers (rounded).
  auto transform = [&](float (&dAcc)[1][4][4], const T *A) {
    FLAB_ACC_FOREACH(1, 4, m0, n32, row, col, mi, ni, r) { dAcc[mi][ni][r] = row > col ? dAcc[mi][ni][r] * sBeta[col] : 0.f; }
    acc_to_smem<1, 4, T>(dAcc, sDA, LDP, m0, n32);
    __syncthreads();
    float x1[1][4][4];
    acc_zero(x1);
    WarpGemm<1, 4, false, false, T>::run(x1, sDA, LDP, m0, A, LDP, n32, C);  // dA A^T
    acc_to_smem<1, 4, T>(x1, sTmp, LDP, m0, n32);
    __syncthreads();
    acc_zero(dAcc);
    WarpGemm<1, 4, true, true, T>::run(dAcc, A, LDP, m0, sTmp, LDP, n32, C);  // A^T (dA A^T)
    FLAB_ACC_FOREACH(1, 4, m0, n32, row, col, mi, ni, r) { dAcc[mi][ni][r] = row > col ? rnd<T>(-dAcc[mi][ni][r]) : 0.f; }
  };

  // optional dk of an earlier stage to accumulate onto: fetched into the v buffer once v is no longer needed
  const T *dk_in = reinterpret_cast<const T *>(a.x);
  auto load_dk_in = [&]() {
    if (dk_in) tile_load<T>(sV, LDX, dk_in + offk, ks, rows, C, a.K, WT, tid, 256);
    cp_async_commit();
  };

  cp_async_wait<1>();
  __syncthreads();  // Aw, k, dw have landed
  if (!GATED) {
    pass(sK, sDW, sAw, a.K, dA);
    cp_async_wait<0>();
    __syncthreads();  // v, du have landed
    pass(sV, sDU, sAw, a.V, dA);
    load_dk_in();
    transform(dA, sAw);
  } else {
    pass(sK, sDW, sAw, a.K, dA);
    transform(dA, sAw);
    cp_async_wait<0>();
    __syncthreads();  // Au, v, du have landed; every warp is done with the staging buffers
    pass(sV, sDU, sAu, a.V, dA2);
    load_dk_in();
    transform(dA2, sAu);
    FLAB_ACC_FOREACH(1, 4, m0, n32, row, col, mi, ni, r) {
      const float x2 = dA2[mi][ni][r] * safe_fexp<T>(sG[row] - sG[col]);
      dA2[mi][ni][r] = x2;
      dA[mi][ni][r] = rnd<T>(dA[mi][ni][r] + x2);
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // dv is complete in sDU; the staging buffers are idle; dk_in has landed
  tile_store<T>(reinterpret_cast<T *>(a.dv) + offv, vs, sDU, LDX, rows, a.V, tid, 256);
  acc_to_smem<1, 4, T>(dA, sDA, LDP, m0, n32);
  {
    float dAb[1][4][4];
    FLAB_ACC_FOREACH(1, 4, m0, n32, row, col, mi, ni, r) { dAb[mi][ni][r] = dA[mi][ni][r] * sBeta[row]; }
    acc_to_smem<1, 4, T>(dAb, sTmp, LDP, m0, n32);
  }
  __syncthreads();

  // dk = (A^T dw) beta + (dA k) beta + (diag(beta) dA)^T k ; dbeta += sum((dA k) * k)
  if (n64 < a.K) {
    float acc[1][8][4];
    acc_zero(acc);
    WarpGemm<1, 8, false, true, T>::run(acc, sDA, LDP, m0, sK, LDX, n64, C);  // dA k
    const float b_lo = sBeta[m0 + g8], b_hi = sBeta[m0 + g8 + 8];
#pragma unroll
    for (int ni = 0; ni < 8; ++ni) {
      const int col = n64 + ni * 8 + 2 * t4;
      const int o_lo = (m0 + g8) * LDX + col, o_hi = (m0 + g8 + 8) * LDX + col;
      const float2 k_lo = ld_pair<T>(sK + o_lo), k_hi = ld_pair<T>(sK + o_hi);
      const float2 d_lo = ld_pair<T>(sDW + o_lo), d_hi = ld_pair<T>(sDW + o_hi);  // first-pass dk (rounded to T)
      dbeta_lo += acc[0][ni][0] * k_lo.x + acc[0][ni][1] * k_lo.y;
      dbeta_hi += acc[0][ni][2] * k_hi.x + acc[0][ni][3] * k_hi.y;
      acc[0][ni][0] = d_lo.x + acc[0][ni][0] * b_lo;
      acc[0][ni][1] = d_lo.y + acc[0][ni][1] * b_lo;
      acc[0][ni][2] = d_hi.x + acc[0][ni][2] * b_hi;
      acc[0][ni][3] = d_hi.y + acc[0][ni][3] * b_hi;
      if (dk_in) {
        const float2 i_lo = ld_pair<T>(sV + o_lo), i_hi = ld_pair<T>(sV + o_hi);
        acc[0][ni][0] += i_lo.x;
        acc[0][ni][1] += i_lo.y;
        acc[0][ni][2] += i_hi.x;
        acc[0][ni][3] += i_hi.y;
      }
    }
    WarpGemm<1, 8, true, true, T>::run(acc, sTmp, LDP, m0, sK, LDX, n64, C);  // (diag(beta) dA)^T k
    // each thread overwrites exactly the sDW elements it just read
    acc_to_smem<1, 8, T>(acc, sDW, LDX, m0, n64);
  }
  // dbeta: quad reduction, then the two column halves meet in shared memory
  dbeta_lo += __shfl_xor_sync(0xffffffffu, dbeta_lo, 1);
  dbeta_lo += __shfl_xor_sync(0xffffffffu, dbeta_lo, 2);
  dbeta_hi += __shfl_xor_sync(0xffffffffu, dbeta_hi, 1);
  dbeta_hi += __shfl_xor_sync(0xffffffffu, dbeta_hi, 2);
  if (t4 == 0) {
    atomicAdd(&sDB[m0 + g8], dbeta_lo);
    atomicAdd(&sDB[m0 + g8 + 8], dbeta_hi);
  }
  if (GATED) {
    // dg = rowsum(dA2 * Gram) - colsum(dA2 * Gram), Gram = diag(beta) k k^T
    float gram[1][4][4];
    acc_zero(gram);
    WarpGemm<1, 4, false, false, T>::run(gram, sK, LDX, m0, sK, LDX, n32, round_up(a.K, 16));
    const float b_lo = sBeta[m0 + g8], b_hi = sBeta[m0 + g8 + 8];
    float r_lo = 0.f, r_hi = 0.f;
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const float p0 = dA2[0][ni][0] * gram[0][ni][0] * b_lo, p1 = dA2[0][ni][1] * gram[0][ni][1] * b_lo;
      const float p2 = dA2[0][ni][2] * gram[0][ni][2] * b_hi, p3 = dA2[0][ni][3] * gram[0][ni][3] * b_hi;
      r_lo += p0 + p1;
      r_hi += p2 + p3;
      float c0 = p0 + p2, c1 = p1 + p3;
      c0 += __shfl_xor_sync(0xffffffffu, c0, 4);
      c0 += __shfl_xor_sync(0xffffffffu, c0, 8);
      c0 += __shfl_xor_sync(0xffffffffu, c0, 16);
      c1 += __shfl_xor_sync(0xffffffffu, c1, 4);
      c1 += __shfl_xor_sync(0xffffffffu, c1, 8);
      c1 += __shfl_xor_sync(0xffffffffu, c1, 16);
      if (g8 == 0) {
        atomicAdd(&sDG[n32 + ni * 8 + 2 * t4], -c0);
        atomicAdd(&sDG[n32 + ni * 8 + 2 * t4 + 1], -c1);
      }
    }
    r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 1);
    r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 2);
    r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 1);
    r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 2);
    if (t4 == 0) {
      atomicAdd(&sDG[m0 + g8], r_lo);
      atomicAdd(&sDG[m0 + g8 + 8], r_hi);
    }
  }
  __syncthreads();
  tile_store<T>(reinterpret_cast<T *>(a.dk) + offk, ks, sDW, LDX, rows, a.K, tid, 256);
  if (tid < rows) {
    reinterpret_cast<float *>(a.dbeta)[tok_off(a, s, hd, t0 + tid, 1)] = sDB[tid];
    if (GATED) reinterpret_cast<float *>(a.dg)[tok_off(a, s, hd, t0 + tid, 1)] = sDG[tid];
  }
}

template <typename T, bool GATED, bool RECOMPUTE> static int launch_wy_fwd(const flab_args *a, cudaStream_t stream) {
  constexpr int LDX = WT + Num<T>::pad, LDP = C + Num<T>::pad, NM = GATED ? 2 : 1;
  if (sizeof(T) == 2 && a->K <= WT && a->V <= WT) {
    size_t smem = ((size_t)2 * C * LDX + (size_t)NM * C * LDP) * sizeof(T) + 2 * C * sizeof(float);
    if (!RECOMPUTE) smem += (size_t)C * LDL * sizeof(float);
    auto kern = wy_fwd16_kernel<T, GATED, RECOMPUTE>;
    if (int e = set_smem(kern, smem)) return e;
    kern<<<dim3(a->NT, a->H), 256, smem, stream>>>(*a);
    return check_launch(RECOMPUTE ? "wy_recompute" : "wy_fwd");
  }
  size_t smem = ((size_t)2 * C * LDX + (size_t)NM * C * LDP) * sizeof(T) + 2 * C * sizeof(float);
  if (!RECOMPUTE) smem += ((size_t)NM * C * LDL + (size_t)NM * 32 * 33) * sizeof(float);
  auto kern = wy_fwd_kernel<T, GATED, RECOMPUTE>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(a->NT, a->H), 128, smem, stream>>>(*a);
  return check_launch(RECOMPUTE ? "wy_recompute" : "wy_fwd");
}

template <typename T, bool GATED> static int launch_wy_bwd(const flab_args *a, cudaStream_t stream) {
  constexpr int LDX = WT + Num<T>::pad, LDP = C + Num<T>::pad;
  if (sizeof(T) == 2 && a->K <= WT && a->V <= WT) {
    size_t smem = ((size_t)4 * C * LDX + (size_t)(GATED ? 4 : 3) * C * LDP) * sizeof(T) + 4 * C * sizeof(float);
    auto kern = wy_bwd16_kernel<T, GATED>;
    if (int e = set_smem(kern, smem)) return e;
    kern<<<dim3(a->NT, a->H), 256, smem, stream>>>(*a);
    return check_launch("wy_bwd");
  }
  size_t smem = ((size_t)3 * C * LDX + (size_t)(GATED ? 4 : 3) * C * LDP) * sizeof(T) + 3 * C * sizeof(float);
  auto kern = wy_bwd_kernel<T, GATED>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(a->NT, a->H), 128, smem, stream>>>(*a);
  return check_launch("wy_bwd");
}

// tcgen05 / TMA kernel for the shapes it covers (tc_wy_bwd.cu); 1 = handled, 0 = not applicable
int tc_wy_bwd_try(const flab_args *a, cudaStream_t stream);
int tc_wy_fwd_try(const flab_args *a, cudaStream_t stream);
static bool tc_wy_enabled() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("FLA_B200_NO_TC");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace flab

namespace flab {
__global__ void add_inplace_kernel(float *__restrict__ x, const float *__restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += y[i];
}
}  // namespace flab

extern "C" {

int flab_wy_fwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->k && a->v && a->beta && a->aw && a->w && a->u, FLAB_E_BADARG, "wy_fwd needs k, v, beta, aw, w and u");
  FLAB_REQUIRE(!a->g || a->au, FLAB_E_BADARG, "wy_fwd: g given but au is NULL");
  if (tc_wy_enabled()) {
    const int r = tc_wy_fwd_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_DISPATCH_16(a->dtype, T, {
    if (a->g) return (launch_wy_fwd<T, true, false>(a, (cudaStream_t)stream));
    return (launch_wy_fwd<T, false, false>(a, (cudaStream_t)stream));
  });
  return FLAB_OK;
}

int flab_wy_recompute(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->k && a->v && a->beta && a->aw && a->w && a->u, FLAB_E_BADARG, "wy_recompute needs k, v, beta, aw, w and u");
  FLAB_DISPATCH_16(a->dtype, T, {
    if (a->au) return (launch_wy_fwd<T, true, true>(a, (cudaStream_t)stream));
    return (launch_wy_fwd<T, false, true>(a, (cudaStream_t)stream));
  });
  return FLAB_OK;
}

int flab_wy_bwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->k && a->v && a->beta && a->aw && a->dw && a->du && a->dk && a->dv && a->dbeta, FLAB_E_BADARG,
               "wy_bwd needs k, v, beta, aw, dw, du, dk, dv and dbeta");
  const bool gated = a->g != nullptr;
  FLAB_REQUIRE(!gated || (a->au && a->dg), FLAB_E_BADARG, "wy_bwd: g given but au or dg is NULL");
  if (tc_wy_enabled()) {
    const int r = tc_wy_bwd_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  int rc = FLAB_OK;
  FLAB_DISPATCH_16(a->dtype, T, {
    rc = gated ? launch_wy_bwd<T, true>(a, (cudaStream_t)stream) : launch_wy_bwd<T, false>(a, (cudaStream_t)stream);
  });
  if (rc != FLAB_OK || !gated || !a->dgk) return rc;
  // these kernels leave dg w.r.t. the cumulative gate; the optional last step (add the dg of the preceding stage, reverse
  // chunk-local cumsum) follows as two small launches: an in-place add, then the cumsum kernel in place
  const long long n = (long long)a->B * a->T * a->H;
  add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<float *>(a->dg),
                                                                                  reinterpret_cast<const float *>(a->dgk), n);
  if (int e = check_launch("wy_bwd(dg add)")) return e;
  flab_args c = *a;
  c.dtype = FLAB_FP32;
  c.flags = FLAB_F_REVERSE;
  c.x = a->dg;
  c.y = a->dg;
  return flab_chunk_local_cumsum_scalar(&c, stream);
}
}
