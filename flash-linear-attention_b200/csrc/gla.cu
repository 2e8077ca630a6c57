// GLA: gates per key channel, b = chunk-local cumsum of the log gates (fp32 [.., K]).
//   fwd_intra : A_ij = scale * sum_k q_ik k_jk e^{b_ik - b_jk}, i >= j          (fla/ops/gla/chunk.py:29-170)
//   fwd_o     : o = (q*scale*e^{b}) h + tril(A) v                                (fla/ops/gla/chunk.py:320-393)
//   bwd_dav   : dA = tril(do v^T) * scale;  dv = tril(A)^T do + (k e^{b_L-b}) dh (fla/ops/gla/chunk.py:583-710)
//   bwd_dqkg  : dq, dk (intra + inter) and dg with the in-chunk reverse cumsum   (fla/ops/gla/chunk.py:409-567, 726-837)
// The gate couples every (i, j, channel) triple, so the intra-chunk terms are not one GEMM with row / column
// scaling.  The gate factors are split at the first row r of each block of 16 rows,
// e^{b_i - b_j} = e^{b_i - b_r} e^{b_r - b_j}: the exponentials are taken once per element and each 16-row block
// becomes one tile product on fp32 operand tiles (TF32 tensor-core path for 16-bit element types - bf16 operands
// are too coarse for dg, a difference of nearly cancelling sums - and plain FMAs for fp32); a block whose decay
// over its 16 tokens would overflow the split takes the direct form.  The state products use the tile GEMM.
// No global load sits between two barriers: inputs of a later phase are copied asynchronously (cp.async) while
// the earlier phase computes, gate rows are fetched into registers before the wait on the tile copies.
#include "common.cuh"

namespace flab {

constexpr int GT = 64;  // key-channel tile of the intra / dqkg kernels

// ------------------------------------------------------------------------------------------------
// A = intra-chunk scores (fp32). grid (NT, H); 256 threads; K walked in tiles of 64 channels.
// The triple (i, j, channel) only couples through e^{b_i - b_j}.  For a block of 16 rows with first row r,
// e^{b_i - b_j} = e^{b_i - b_r} e^{b_r - b_j}: both factors are applied once per element, which leaves one tile
// product per 16 x 16 block of A (TF32 tensor-core path for 16-bit element types, plain FMAs for fp32).  For j
// before the block the second exponent is <= 0.  Inside the block it is positive but bounded by the decay over 16
// tokens; when that exceeds e^60 in some channel (never with gates from a log-sigmoid) the diagonal block is
// evaluated directly instead.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256, 2) gla_fwd_intra_kernel(const flab_args a) {
  constexpr int LDF = GT + 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float *stB = reinterpret_cast<float *>(smem_raw);  // [64][64] gates of the channel tile, as copied
  float *tQs = stB + C * GT;                          // [64][LDF] q re-based to the first row of its row block
  float *tKF = tQs + C * LDF;                         // [16+32+48+64][LDF] k re-based to the first row of block I, stacked
  T *stQ = reinterpret_cast<T *>(tKF + 160 * LDF);    // [64][64] q, k of the channel tile, as copied
  T *stK = stQ + C * GT;
  __shared__ int sDirect[2][4];
  const int tid = threadIdx.x, warp = tid >> 5;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0);
  const size_t ks = tok_stride(a, a.K), offk = tok_off(a, s, hd, t0, a.K);
  const T *q = reinterpret_cast<const T *>(a.q) + offk, *k = reinterpret_cast<const T *>(a.k) + offk;
  const float *b = reinterpret_cast<const float *>(a.gk) + offk;
  // the ten 16 x 16 blocks (I, m <= I) on and below the diagonal: warp w owns block w, warps 0 and 1 also 8 and 9
  const int nblk = warp < 2 ? 2 : 1;
  int bI[2], bM[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int id = warp + 8 * x;
    const int I = id < 1 ? 0 : id < 3 ? 1 : id < 6 ? 2 : 3;
    bI[x] = I;
    bM[x] = id - I * (I + 1) / 2;
  }
  float acc[2][1][2][4];
  acc_zero(acc[0]);
  acc_zero(acc[1]);
  // the channel tile's inputs are copied asynchronously; the copy of the next tile runs under the products of this one
  auto stage = [&](int k0) {
    const int kw = min(GT, a.K - k0);
    tile_load<T>(stQ, GT, q + k0, ks, rows, C, kw, GT, tid, 256);
    tile_load<T>(stK, GT, k + k0, ks, rows, C, kw, GT, tid, 256);
    tile_load<float>(stB, GT, b + k0, ks, rows, C, kw, GT, tid, 256);
    cp_async_commit();
  };
  stage(0);
  for (int k0 = 0, tile = 0; k0 < a.K; k0 += GT, ++tile) {
    const int kw = min(GT, a.K - k0);
    int *direct = sDirect[tile & 1];
    if (tid < 4) direct[tid] = 0;
    cp_async_wait<0>();
    __syncthreads();  // tile landed; the products of the previous tile are done with tQs / tKF
    if (tid < GT) {
#pragma unroll
      for (int I = 0; I < 4; ++I) {
        const int r0 = 16 * I, rend = min(r0 + 16, rows);
        if (r0 < rows && stB[r0 * GT + tid] - stB[(rend - 1) * GT + tid] > 60.f) direct[I] = 1;
      }
    }
#pragma unroll
    for (int p = 0; p < C * GT / 256; ++p) {
      const int e = tid + 256 * p, r = e / GT, c = e - r * GT;
      tQs[r * LDF + c] = tile_round<T>(Num<T>::f(stQ[e]) * fexp<T>(stB[e] - stB[(r & ~15) * GT + c]));
    }
    __syncthreads();
#pragma unroll
    for (int I = 0; I < 4; ++I) {
      const int r0 = 16 * I;
      if (r0 >= rows) break;  // uniform
      const int jend = direct[I] ? r0 : min(r0 + 16, rows);
      float *dst = tKF + 8 * I * (I + 1) * LDF;
      for (int e = tid; e < (r0 + 16) * GT; e += 256) {
        const int r = e / GT, c = e - r * GT;
        dst[r * LDF + c] = r < jend ? tile_round<T>(Num<T>::f(stK[e]) * fexp<T>(stB[r0 * GT + c] - stB[e])) : 0.f;
      }
    }
    __syncthreads();  // operand tiles complete, the copied tile is free
    if (k0 + GT < a.K) stage(k0 + GT);
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      if (x >= nblk) break;
      const int I = bI[x], m = bM[x], r0 = 16 * I;
      if (r0 >= rows) continue;
      gemm_f32tile<1, 2, false, false, T>(acc[x], tQs, LDF, r0, tKF + 8 * I * (I + 1) * LDF, LDF, 16 * m, GT);
      if (m == I && direct[I]) {
        FLAB_ACC_FOREACH(1, 2, r0, 16 * m, row, col, mi, ni, r) {
          if (row < rows && col <= row) {
            const T *qi = q + (size_t)row * ks + k0, *kj = k + (size_t)col * ks + k0;
            const float *bi = b + (size_t)row * ks + k0, *bj = b + (size_t)col * ks + k0;
            float v = 0.f;
            for (int c = 0; c < kw; ++c) v = fmaf(Num<T>::f(qi[c]) * Num<T>::f(kj[c]), fexp<T>(bi[c] - bj[c]), v);
            acc[x][mi][ni][r] += v;
          }
        }
      }
    }
  }
  float *A = reinterpret_cast<float *>(a.a) + tok_off(a, s, hd, t0, C);
  const size_t as_ = tok_stride(a, C);
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    if (x >= nblk) break;
    const int I = bI[x], m = bM[x];
    FLAB_ACC_FOREACH(1, 2, 16 * I, 16 * m, row, col, mi, ni, r) {
      if (row < rows) A[(size_t)row * as_ + col] = col <= row ? acc[x][mi][ni][r] * a.scale : 0.f;
    }
  }
  // the six blocks above the diagonal are zero
  for (int e = tid; e < 6 * 256; e += 256) {
    const int id = e >> 8, w = e & 255, I = id < 3 ? 0 : id < 5 ? 1 : 2;
    const int m = I + 1 + (id - (I == 0 ? 0 : I == 1 ? 3 : 5));
    const int row = 16 * I + (w >> 4), col = 16 * m + (w & 15);
    if (row < rows) A[(size_t)row * as_ + col] = 0.f;
  }
}

// Gate factors of a [rows][K] operand tile, eight channels per thread and pass.  GateRows::fetch issues the global
// loads of the gate rows (registers) so that they overlap the tile copies in flight; apply() rescales the tile in
// shared memory once it has landed.  MODE 0: x <- round(x * scale) * e^{b_r};  MODE 1: x <- x * e^{b_last - b_r}.
// Covers K in {8, 16, 32, 64, 128} with 16-byte aligned gate rows; usable() is false otherwise (scalar loop).
template <typename T, int MODE> struct GateRows {
  float4 bv[8][2], bl[2];
  int cpr, c;
  static __device__ __forceinline__ bool usable(const flab_args &a, const float *b, size_t ks) {
    const int cpr = a.K >> 3;
    return a.K % 8 == 0 && a.K <= 128 && cpr > 0 && 128 % cpr == 0 && ((uintptr_t)b) % 16 == 0 && (ks * sizeof(float)) % 16 == 0;
  }
  __device__ __forceinline__ void fetch(const flab_args &a, const float *b, size_t ks, int rows, int tid) {
    cpr = a.K >> 3;
    c = (tid % cpr) * 8;  // 128 % cpr == 0: the channel group of a thread is the same in every pass
    const int rstep = 128 / cpr, r0 = tid / cpr;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = r0 + u * rstep;
      if (r < rows) {
        bv[u][0] = *reinterpret_cast<const float4 *>(b + (size_t)r * ks + c);
        bv[u][1] = *reinterpret_cast<const float4 *>(b + (size_t)r * ks + c + 4);
      } else {
        bv[u][0] = bv[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    if (MODE == 1) {
      bl[0] = *reinterpret_cast<const float4 *>(b + (size_t)(rows - 1) * ks + c);
      bl[1] = *reinterpret_cast<const float4 *>(b + (size_t)(rows - 1) * ks + c + 4);
    } else {
      bl[0] = bl[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  __device__ __forceinline__ void apply(T *x, int ld, int rows, float scale, int tid) const {
    const int rstep = 128 / cpr, r0 = tid / cpr;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = r0 + u * rstep;
      if (r >= rows) continue;
      T *px = x + r * ld + c;
      const float g[8] = {bv[u][0].x, bv[u][0].y, bv[u][0].z, bv[u][0].w, bv[u][1].x, bv[u][1].y, bv[u][1].z, bv[u][1].w};
      const float l[8] = {bl[0].x, bl[0].y, bl[0].z, bl[0].w, bl[1].x, bl[1].y, bl[1].z, bl[1].w};
      T v[8];
      if constexpr (sizeof(T) == 2) *reinterpret_cast<int4 *>(v) = *reinterpret_cast<const int4 *>(px);
      else {
        *reinterpret_cast<int4 *>(v) = *reinterpret_cast<const int4 *>(px);
        *reinterpret_cast<int4 *>(v + 4) = *reinterpret_cast<const int4 *>(px + 4);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xf = Num<T>::f(v[j]);
        v[j] = Num<T>::t(MODE == 0 ? rnd<T>(xf * scale) * expf(g[j]) : xf * expf(l[j] - g[j]));
      }
      if constexpr (sizeof(T) == 2) *reinterpret_cast<int4 *>(px) = *reinterpret_cast<const int4 *>(v);
      else {
        *reinterpret_cast<int4 *>(px) = *reinterpret_cast<const int4 *>(v);
        *reinterpret_cast<int4 *>(px + 4) = *reinterpret_cast<const int4 *>(v + 4);
      }
    }
  }
};

// tril(A) (fp32 [64][64] in global memory) -> operand tile of type T, four columns per thread and pass
template <typename T> __device__ __forceinline__ void load_tril_A(T *sA, int ldp, const float *A, size_t as_, int rows, int tid) {
  if (((uintptr_t)A) % 16 == 0 && (as_ * sizeof(float)) % 16 == 0) {
#pragma unroll
    for (int u = 0; u < C * C / 4 / 128; ++u) {
      const int e = tid + 128 * u, i = e >> 4, j = (e & 15) * 4;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < rows && j <= i) x = *reinterpret_cast<const float4 *>(A + (size_t)i * as_ + j);
      sA[i * ldp + j] = Num<T>::t(x.x);
      sA[i * ldp + j + 1] = Num<T>::t(j + 1 <= i ? x.y : 0.f);
      sA[i * ldp + j + 2] = Num<T>::t(j + 2 <= i ? x.z : 0.f);
      sA[i * ldp + j + 3] = Num<T>::t(j + 3 <= i ? x.w : 0.f);
    }
  } else {
    for (int e = tid; e < C * C; e += 128) {
      int i = e >> 6, j = e & 63;
      sA[i * ldp + j] = Num<T>::t((i < rows && i >= j) ? A[(size_t)i * as_ + j] : 0.f);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// o = (q*scale*e^{b}) h + tril(A) v.  grid (NT, H, V/BV); 4 warps x 16 token rows.
// ------------------------------------------------------------------------------------------------
template <typename T, int BV>
__global__ void __launch_bounds__(128) gla_fwd_o_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KP = round_up(a.K, 16);
  const int LDK = KP + Num<T>::pad;
  constexpr int LDV = BV + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  T *sQ = reinterpret_cast<T *>(smem_raw);  // [64][LDK] q -> q*scale*e^{b}
  T *sV = sQ + C * LDK;                     // [64][LDV]; reused to stage o
  T *sA = sV + C * LDV;                     // [64][LDP]
  T *sH = sA + C * LDP;                     // [KP][LDV]
  const int tid = threadIdx.x, warp = tid >> 5;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y, v0 = blockIdx.z * BV;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0), vw = min(BV, a.V - v0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V) + v0;
  tile_load<T>(sQ, LDK, reinterpret_cast<const T *>(a.q) + offk, ks, rows, C, a.K, KP, tid, 128);
  tile_load<T>(sV, LDV, reinterpret_cast<const T *>(a.v) + offv, vs, rows, C, vw, BV, tid, 128);
  tile_load<T>(sH, LDV, reinterpret_cast<const T *>(a.h) + ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + v0, (size_t)a.V,
               a.K, KP, vw, BV, tid, 128);
  cp_async_commit();
  const float *b = reinterpret_cast<const float *>(a.gk) + offk;
  GateRows<T, 0> gates;
  const bool gvec = GateRows<T, 0>::usable(a, b, ks);
  if (gvec) gates.fetch(a, b, ks, rows, tid);
  load_tril_A<T>(sA, LDP, reinterpret_cast<const float *>(a.a) + tok_off(a, s, hd, t0, C), as_, rows, tid);
  cp_async_wait<0>();
  __syncthreads();
  if (gvec) {
    gates.apply(sQ, LDK, rows, a.scale, tid);
  } else {
    for (int e = tid; e < rows * a.K; e += 128) {
      int r = e / a.K, c = e - r * a.K;
      float x = rnd<T>(Num<T>::f(sQ[r * LDK + c]) * a.scale) * expf(b[(size_t)r * ks + c]);
      sQ[r * LDK + c] = Num<T>::t(x);
    }
  }
  __syncthreads();
  constexpr int NI = BV / 8;
  const int m0 = warp * 16;
  float acc[1][NI][4];
  acc_zero(acc);
  WarpGemm<1, NI, false, true, T>::run(acc, sQ, LDK, m0, sH, LDV, 0, KP);
  WarpGemm<1, NI, false, true, T>::run(acc, sA, LDP, m0, sV, LDV, 0, C);
  __syncthreads();
  acc_to_smem<1, NI, T>(acc, sV, LDV, m0, 0);
  __syncthreads();
  tile_store<T>(reinterpret_cast<T *>(a.o) + offv, vs, sV, LDV, rows, vw, tid, 128);
}

// ------------------------------------------------------------------------------------------------
// dA and dv.  grid (NT, H, V/BV).  Every V tile recomputes nothing shared: dA needs the full V
// contraction, so it is computed by the CTA of V tile 0 over all of V; dv per V tile.
// ------------------------------------------------------------------------------------------------
template <typename T, int BV>
__global__ void __launch_bounds__(128) gla_bwd_dav_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KP = round_up(a.K, 16);
  const int LDK = KP + Num<T>::pad;
  constexpr int LDV = BV + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  T *sKG = reinterpret_cast<T *>(smem_raw);  // [64][LDK] k * e^{b_L - b}
  T *sDO = sKG + C * LDK;                    // [64][LDV]; reused to stage dv
  T *sVV = sDO + C * LDV;                    // [64][LDV] v tile (dA only)
  T *sA = sVV + C * LDV;                     // [64][LDP]
  T *sDH = sA + C * LDP;                     // [KP][LDV]
  const int tid = threadIdx.x, warp = tid >> 5;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y, v0 = blockIdx.z * BV;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0), last = rows - 1, vw = min(BV, a.V - v0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv0 = tok_off(a, s, hd, t0, a.V);
  const int m0 = warp * 16;

  // dA = tril(do v^T) * scale over all V tiles (CTA with blockIdx.z == 0 only)
  if (blockIdx.z == 0) {
    float dA[1][8][4];
    acc_zero(dA);
    for (int c0 = 0; c0 < a.V; c0 += BV) {
      const int cw = min(BV, a.V - c0);
      __syncthreads();
      tile_load<T>(sDO, LDV, reinterpret_cast<const T *>(a.d_o) + offv0 + c0, vs, rows, C, cw, BV, tid, 128);
      tile_load<T>(sVV, LDV, reinterpret_cast<const T *>(a.v) + offv0 + c0, vs, rows, C, cw, BV, tid, 128);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      WarpGemm<1, 8, false, false, T>::run(dA, sDO, LDV, m0, sVV, LDV, 0, BV);
    }
    float *dAo = reinterpret_cast<float *>(a.da) + tok_off(a, s, hd, t0, C);
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) {
      if (row < rows) dAo[(size_t)row * as_ + col] = row >= col ? dA[mi][ni][r] * a.scale : 0.f;
    }
    __syncthreads();
  }
  tile_load<T>(sKG, LDK, reinterpret_cast<const T *>(a.k) + offk, ks, rows, C, a.K, KP, tid, 128);
  tile_load<T>(sDO, LDV, reinterpret_cast<const T *>(a.d_o) + offv0 + v0, vs, rows, C, vw, BV, tid, 128);
  tile_load<T>(sDH, LDV, reinterpret_cast<const T *>(a.dh) + ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + v0, (size_t)a.V,
               a.K, KP, vw, BV, tid, 128);
  cp_async_commit();
  const float *b = reinterpret_cast<const float *>(a.gk) + offk;
  GateRows<T, 1> gates;
  const bool gvec = GateRows<T, 1>::usable(a, b, ks);
  if (gvec) gates.fetch(a, b, ks, rows, tid);
  load_tril_A<T>(sA, LDP, reinterpret_cast<const float *>(a.a) + tok_off(a, s, hd, t0, C), as_, rows, tid);
  cp_async_wait<0>();
  __syncthreads();
  if (gvec) {
    gates.apply(sKG, LDK, rows, 1.f, tid);
  } else {
    for (int e = tid; e < rows * a.K; e += 128) {
      int r = e / a.K, c = e - r * a.K;
      float x = Num<T>::f(sKG[r * LDK + c]) * expf(b[(size_t)last * ks + c] - b[(size_t)r * ks + c]);
      sKG[r * LDK + c] = Num<T>::t(x);
    }
  }
  __syncthreads();
  constexpr int NI = BV / 8;
  float acc[1][NI][4];
  acc_zero(acc);
  WarpGemm<1, NI, true, true, T>::run(acc, sA, LDP, m0, sDO, LDV, 0, C);   // tril(A)^T do
  WarpGemm<1, NI, false, true, T>::run(acc, sKG, LDK, m0, sDH, LDV, 0, KP);  // (k e^{b_L-b}) dh
  __syncthreads();
  acc_to_smem<1, NI, T>(acc, sDO, LDV, m0, 0);
  __syncthreads();
  tile_store<T>(reinterpret_cast<T *>(a.dv) + offv0 + v0, vs, sDO, LDV, rows, vw, tid, 128);
}

// ------------------------------------------------------------------------------------------------
// dq, dk, dg.  grid (NT, H, K/64); 256 threads = 8 warps, warp (rb, ch) owns rows 16 rb .. and channels 32 ch .. of
// the chunk's [64][64] dq and dk tiles in mma fragments, from the first product to the last.
// Phase 1: inter-chunk products (do h^T, v dh^T).  Phase 2: intra-chunk terms as tile products on fp32 operand
// tiles (TF32 tensor-core path for 16-bit element types, plain FMAs for fp32), with the per-channel gates split
// per block of 16 rows: e^{b_i - b_j} = e^{b_i - b_r} e^{b_r - b_j}, r the block's first row.
//   dq_i  = e^{b_i - b_r} sum_j dA_ij (k_j e^{b_r - b_j})          one product per row block I against KF_I
//   dk_j  = sum_I e^{b_rI - b_j} sum_{i in I} dA_ij (q_i e^{b_i - b_rI})
// For j before the block the exponent b_r - b_j is <= 0; inside the block it is bounded by the decay over 16
// tokens, and a block where that exceeds e^60 in some channel evaluates its in-block pairs directly.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gla_bwd_dqkg_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int VP = round_up(a.V, 16);
  const int LDV = VP + Num<T>::pad;
  constexpr int LD = GT + 1;   // column-walk tiles
  constexpr int LDF = GT + 4;  // mma operand tiles (fragment loads conflict-free)
  float *sGK = reinterpret_cast<float *>(smem_raw);  // [64] per-channel chunk term of dg
  int *sDirect = reinterpret_cast<int *>(sGK + GT);  // [4] row block evaluates its in-block pairs directly
  unsigned char *region = reinterpret_cast<unsigned char *>(sDirect + 4);
  // phase 1 view
  T *sDO = reinterpret_cast<T *>(region);  // [64][LDV]
  T *sVV = sDO + C * LDV;                  // [64][LDV]
  T *sH = sVV + C * LDV;                   // [64 channels][LDV]
  T *sDH = sH + GT * LDV;                  // [64 channels][LDV]
  // phase 2 view
  float *sK = reinterpret_cast<float *>(region);  // [64][LD]
  float *sB = sK + C * LD;                        // [64][LD]
  float *tDA = sB + C * LD;                       // [64][LDF] tril(dA)
  float *tQs = tDA + C * LDF;                     // [64][LDF] q re-based to the first row of its row block
  float *tKF = tQs + C * LDF;                     // [16+32+48+64][LDF] k re-based to the first row of block I, stacked
  float *sOQ = tKF;                               // [64][LD] total dq (after the products)
  // staging of the phase-2 inputs, fetched while phase 1 runs: behind the phase-1 tiles, inside what becomes tKF
  const size_t p1_bytes = ((size_t)2 * C * LDV + (size_t)2 * GT * LDV) * sizeof(T);
  const size_t p2_bytes = ((size_t)2 * C * LD + (size_t)(2 * C + 160) * LDF) * sizeof(float);
  constexpr size_t STG_BYTES = (size_t)2 * C * GT * sizeof(T) + (size_t)(C * GT + 10 * 256) * sizeof(float);
  const size_t stg_off = p1_bytes + STG_BYTES > p2_bytes ? p1_bytes : p2_bytes - STG_BYTES;
  float *stB = reinterpret_cast<float *>(region + ((stg_off + 15) & ~(size_t)15));  // [64][64] gates
  float *stDA = stB + C * GT;                     // [10][16][16] blocks (I, m <= I) of dA
  T *stQ = reinterpret_cast<T *>(stDA + 10 * 256);  // [64][64]
  T *stK = stQ + C * GT;                          // [64][64]
  float *sOK = sOQ + C * LD;                      // [64][LD] total dk

  const int tid = threadIdx.x, warp = tid >> 5;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y, k0 = blockIdx.z * GT;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0), last = rows - 1, kw = min(GT, a.K - k0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K) + k0, offv = tok_off(a, s, hd, t0, a.V);
  const float *b = reinterpret_cast<const float *>(a.gk) + offk;
  const int rb = warp & 3, ch = warp >> 2, m0 = rb * 16, n0 = ch * 32;
  float dq[1][4][4], dk[1][4][4];

  // ---- phase 1
  {
    const size_t hoff = ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + (size_t)k0 * a.V;
    tile_load<T>(sDO, LDV, reinterpret_cast<const T *>(a.d_o) + offv, vs, rows, C, a.V, VP, tid, 256);
    tile_load<T>(sVV, LDV, reinterpret_cast<const T *>(a.v) + offv, vs, rows, C, a.V, VP, tid, 256);
    tile_load<T>(sH, LDV, reinterpret_cast<const T *>(a.h) + hoff, (size_t)a.V, kw, GT, a.V, VP, tid, 256);
    tile_load<T>(sDH, LDV, reinterpret_cast<const T *>(a.dh) + hoff, (size_t)a.V, kw, GT, a.V, VP, tid, 256);
    cp_async_commit();
    {
      const float *dA = reinterpret_cast<const float *>(a.da) + tok_off(a, s, hd, t0, C);
      tile_load<T>(stQ, GT, reinterpret_cast<const T *>(a.q) + offk, ks, rows, C, kw, GT, tid, 256);
      tile_load<T>(stK, GT, reinterpret_cast<const T *>(a.k) + offk, ks, rows, C, kw, GT, tid, 256);
      tile_load<float>(stB, GT, b, ks, rows, C, kw, GT, tid, 256);
      {  // one 16 x 16 block of dA per group of 64 threads and pass
        const int grp = tid >> 6, w = tid & 63;
        for (int id = grp; id < 10; id += 4) {
          const int I = id < 1 ? 0 : id < 3 ? 1 : id < 6 ? 2 : 3, m = id - I * (I + 1) / 2;
          tile_load<float>(stDA + id * 256, 16, dA + (size_t)(16 * I) * as_ + 16 * m, as_, max(0, min(16, rows - 16 * I)), 16, 16, 16, w, 64);
        }
      }
      cp_async_commit();
    }
    if (tid < 4) sDirect[tid] = 0;
    cp_async_wait<1>();
    __syncthreads();
    acc_zero(dq);
    acc_zero(dk);
    WarpGemm<1, 4, false, false, T>::run(dq, sDO, LDV, m0, sH, LDV, n0, VP);
    WarpGemm<1, 4, false, false, T>::run(dk, sVV, LDV, m0, sDH, LDV, n0, VP);
    // per-channel sum_v h * dh: four threads per channel
    {
      const int c = tid >> 2, sl = tid & 3;
      float x = 0.f;
      if (c < kw)
        for (int v = sl; v < a.V; v += 4) x = fmaf(Num<T>::f(sH[c * LDV + v]), Num<T>::f(sDH[c * LDV + v]), x);
      x += __shfl_xor_sync(0xffffffffu, x, 1);
      x += __shfl_xor_sync(0xffffffffu, x, 2);
      if (sl == 0) sGK[c] = c < kw ? x * expf(b[(size_t)last * ks + c]) : 0.f;
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // ---- phase 2
  {
    const T *q = reinterpret_cast<const T *>(a.q) + offk;
    float qreg[C * GT / 256];  // q of element e = tid + 256 p (row e / 64, channel e % 64): row block I owns p = 4 I .. 4 I + 3
#pragma unroll
    for (int p = 0; p < C * GT / 256; ++p) {
      const int e = tid + 256 * p, r = e / GT, c = e - r * GT;
      const bool ok = r < rows && c < kw;
      qreg[p] = ok ? Num<T>::f(stQ[e]) : 0.f;
      sK[r * LD + c] = ok ? Num<T>::f(stK[e]) : 0.f;
      sB[r * LD + c] = ok ? stB[e] : 0.f;
      const int I = r >> 4, m = c >> 4;  // c = column of dA here
      tDA[r * LDF + c] = (r < rows && c <= r) ? tile_round<T>(stDA[(I * (I + 1) / 2 + m) * 256 + (r & 15) * 16 + (c & 15)]) : 0.f;
    }
    __syncthreads();
    if (tid < GT) {
#pragma unroll
      for (int I = 0; I < 4; ++I) {
        const int r0 = 16 * I, rend = min(r0 + 16, rows);
        if (r0 < rows && sB[r0 * LD + tid] - sB[(rend - 1) * LD + tid] > 60.f) sDirect[I] = 1;
      }
    }
    {  // gates of the inter-chunk terms; sum_j dk_inter k per channel (before the intra terms are added)
      float part[4][2];
      FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
        const float bi = sB[row * LD + col];
        const bool ok = row < rows && col < kw;
        dq[mi][ni][r] *= ok ? expf(bi) * a.scale : 0.f;
        dk[mi][ni][r] *= ok ? expf(sB[last * LD + col] - bi) : 0.f;
        const float x = dk[mi][ni][r] * sK[row * LD + col];
        if (r < 2) part[ni][r] = x;
        else part[ni][r - 2] += x;
      }
      const int lane = tid & 31;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float x = part[ni][h2];
          x += __shfl_xor_sync(0xffffffffu, x, 4);
          x += __shfl_xor_sync(0xffffffffu, x, 8);
          x += __shfl_xor_sync(0xffffffffu, x, 16);
          if (lane < 4) atomicAdd(&sGK[n0 + 8 * ni + 2 * lane + h2], x);
        }
    }
    __syncthreads();
    // operand tiles
#pragma unroll
    for (int p = 0; p < C * GT / 256; ++p) {
      const int e = tid + 256 * p, r = e / GT, c = e - r * GT;
      tQs[r * LDF + c] = tile_round<T>(qreg[p] * fexp<T>(sB[r * LD + c] - sB[(r & ~15) * LD + c]));
    }
#pragma unroll
    for (int I = 0; I < 4; ++I) {
      const int r0 = 16 * I;
      if (r0 >= rows) break;  // uniform
      const int jend = sDirect[I] ? r0 : min(r0 + 16, rows);
      float *dst = tKF + 8 * I * (I + 1) * LDF;
      for (int e = tid; e < (r0 + 16) * GT; e += 256) {
        const int r = e / GT, c = e - r * GT;
        dst[r * LDF + c] = r < jend ? tile_round<T>(sK[r * LD + c] * fexp<T>(sB[r0 * LD + c] - sB[r * LD + c])) : 0.f;
      }
    }
    __syncthreads();
    // dq of row block rb
    if (m0 < rows) {
      const bool direct = sDirect[rb] != 0;
      float acc[1][4][4];
      acc_zero(acc);
      gemm_f32tile<1, 4, false, true, T>(acc, tDA, LDF, m0, tKF + 8 * rb * (rb + 1) * LDF, LDF, n0, m0 + 16);
      FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
        const float bi = sB[row * LD + col];
        float val = acc[mi][ni][r] * fexp<T>(bi - sB[m0 * LD + col]);
        if (direct && row < rows)
          for (int j = m0; j <= row; ++j) val = fmaf(tDA[row * LDF + j] * sK[j * LD + col], fexp<T>(bi - sB[j * LD + col]), val);
        dq[mi][ni][r] += val;
      }
    }
    // dk of rows 16 rb ..: contributions of every row block I >= rb
    for (int I = rb; I < 4; ++I) {
      const int r0 = 16 * I, rend = min(r0 + 16, rows);
      if (r0 >= rows) break;
      if (I == rb && sDirect[I]) {
        FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
          if (row < rend && col < kw) {
            float x = 0.f;
            for (int i2 = row; i2 < rend; ++i2)
              x = fmaf(tDA[i2 * LDF + row] * Num<T>::f(q[(size_t)i2 * ks + col]), fexp<T>(sB[i2 * LD + col] - sB[row * LD + col]), x);
            dk[mi][ni][r] += x;
          }
        }
        continue;
      }
      float acc[1][4][4];
      acc_zero(acc);
      gemm_f32tile<1, 4, true, true, T>(acc, tDA + r0 * LDF, LDF, m0, tQs + r0 * LDF, LDF, n0, 16);
      FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
        dk[mi][ni][r] = fmaf(acc[mi][ni][r], fexp<T>(sB[r0 * LD + col] - sB[row * LD + col]), dk[mi][ni][r]);
      }
    }
    __syncthreads();
    FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
      sOQ[row * LD + col] = dq[mi][ni][r];
      sOK[row * LD + col] = dk[mi][ni][r];
    }
    __syncthreads();
    // outputs; dg = reverse in-chunk cumsum of (q dq - k dk) + per-channel chunk term
    T *dqo = reinterpret_cast<T *>(a.dq) + offk, *dko = reinterpret_cast<T *>(a.dk) + offk;
#pragma unroll
    for (int p = 0; p < C * GT / 256; ++p) {
      const int e = tid + 256 * p, r = e / GT, c = e - r * GT;
      const float dqv = sOQ[r * LD + c], dkv = sOK[r * LD + c];
      if (r < rows && c < kw) {
        dqo[(size_t)r * ks + c] = Num<T>::t(dqv);
        dko[(size_t)r * ks + c] = Num<T>::t(dkv);
      }
      sOQ[r * LD + c] = qreg[p] * dqv - sK[r * LD + c] * dkv;  // the integrand of dg
    }
    __syncthreads();
    if (tid < kw) {
      float *dg = reinterpret_cast<float *>(a.dgk) + offk;
      float run = sGK[tid];
      for (int r = rows - 1; r >= 0; --r) {
        run += sOQ[r * LD + tid];
        dg[(size_t)r * ks + tid] = run;
      }
    }
  }
}

template <typename T, int BV> static size_t gla_o_smem(const flab_args *a, bool dav) {
  const int KP = round_up(a->K, 16), LDK = KP + Num<T>::pad, LDV = BV + Num<T>::pad, LDP = C + Num<T>::pad;
  size_t e = (size_t)C * LDK + (size_t)C * LDV * (dav ? 2 : 1) + (size_t)C * LDP + (size_t)KP * LDV;
  return e * sizeof(T);
}

template <typename T> static int launch_gla_fwd_intra(const flab_args *a, cudaStream_t stream) {
  size_t smem = ((size_t)C * GT + (size_t)(C + 160) * (GT + 4)) * sizeof(float) + (size_t)2 * C * GT * sizeof(T);
  auto kern = gla_fwd_intra_kernel<T>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(a->NT, a->H), 256, smem, stream>>>(*a);
  return check_launch("gla_fwd_intra");
}

template <typename T> static int launch_gla_fwd_o(const flab_args *a, cudaStream_t stream) {
  if (a->V > 64) {
    auto kern = gla_fwd_o_kernel<T, 128>;
    size_t smem = gla_o_smem<T, 128>(a, false);
    if (int e = set_smem(kern, smem)) return e;
    kern<<<dim3(a->NT, a->H, cdiv(a->V, 128)), 128, smem, stream>>>(*a);
  } else {
    auto kern = gla_fwd_o_kernel<T, 64>;
    size_t smem = gla_o_smem<T, 64>(a, false);
    if (int e = set_smem(kern, smem)) return e;
    kern<<<dim3(a->NT, a->H, 1), 128, smem, stream>>>(*a);
  }
  return check_launch("gla_fwd_o");
}

template <typename T> static int launch_gla_bwd_dav(const flab_args *a, cudaStream_t stream) {
  if (a->V > 64 && sizeof(T) == 2) {
    auto kern = gla_bwd_dav_kernel<T, 128>;
    size_t smem = gla_o_smem<T, 128>(a, true);
    if (int e = set_smem(kern, smem)) return e;
    kern<<<dim3(a->NT, a->H, cdiv(a->V, 128)), 128, smem, stream>>>(*a);
  } else {
    auto kern = gla_bwd_dav_kernel<T, 64>;
    size_t smem = gla_o_smem<T, 64>(a, true);
    if (int e = set_smem(kern, smem)) return e;
    kern<<<dim3(a->NT, a->H, cdiv(a->V, 64)), 128, smem, stream>>>(*a);
  }
  return check_launch("gla_bwd_dav");
}

template <typename T> static int launch_gla_bwd_dqkg(const flab_args *a, cudaStream_t stream) {
  const int VP = round_up(a->V, 16), LDV = VP + Num<T>::pad;
  size_t p1 = ((size_t)2 * C * LDV + (size_t)2 * GT * LDV) * sizeof(T);
  size_t p2 = ((size_t)2 * C * (GT + 1) + (size_t)(2 * C + 160) * (GT + 4)) * sizeof(float);
  size_t stg = (size_t)2 * C * GT * sizeof(T) + (size_t)(C * GT + 10 * 256) * sizeof(float);  // phase-2 inputs staged during phase 1
  size_t stg_off = p1 + stg > p2 ? p1 : p2 - stg;
  size_t smem = (GT + 4) * sizeof(float) + ((stg_off + 15) & ~(size_t)15) + stg;
  auto kern = gla_bwd_dqkg_kernel<T>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(a->NT, a->H, cdiv(a->K, GT)), 256, smem, stream>>>(*a);
  return check_launch("gla_bwd_dqkg");
}

}  // namespace flab

extern "C" {

int flab_gla_fwd_intra(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->gk && a->a, FLAB_E_BADARG, "gla_fwd_intra needs q, k, gk and a");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_gla_fwd_intra<T>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_gla_fwd_o(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->v && a->gk && a->h && a->a && a->o, FLAB_E_BADARG, "gla_fwd_o needs q, v, gk, h, a and o");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_gla_fwd_o<T>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_gla_bwd_dav(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->k && a->v && a->gk && a->a && a->d_o && a->dh && a->da && a->dv, FLAB_E_BADARG,
               "gla_bwd_dav needs k, v, gk, a, d_o, dh, da and dv");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_gla_bwd_dav<T>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_gla_bwd_dqkg(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->gk && a->h && a->dh && a->d_o && a->da && a->dq && a->dk && a->dgk, FLAB_E_BADARG,
               "gla_bwd_dqkg needs q, k, v, gk, h, dh, d_o, da, dq, dk and dgk");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_gla_bwd_dqkg<T>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}
}
