// GLA: gates per key channel, b = chunk-local cumsum of the log gates (fp32 [.., K]).
//   fwd_intra : A_ij = scale * sum_k q_ik k_jk e^{b_ik - b_jk}, i >= j          (fla/ops/gla/chunk.py:29-170)
//   fwd_o     : o = (q*scale*e^{b}) h + tril(A) v                                (fla/ops/gla/chunk.py:320-393)
//   bwd_dav   : dA = tril(do v^T) * scale;  dv = tril(A)^T do + (k e^{b_L-b}) dh (fla/ops/gla/chunk.py:583-710)
//   bwd_dqkg  : dq, dk (intra + inter) and dg with the in-chunk reverse cumsum   (fla/ops/gla/chunk.py:409-567, 726-837)
// The gate couples every (i, j, k) triple, so the intra-chunk terms cannot be factored into one
// GEMM with row/column scaling; they are evaluated directly in fp32 (exponents are always <= 0, so
// nothing overflows and no re-basing is needed).  The state products use the tile GEMM.
#include "common.cuh"

namespace flab {

constexpr int GT = 64;  // key-channel tile of the intra / dqkg kernels

// ------------------------------------------------------------------------------------------------
// A = intra-chunk scores (fp32). grid (NT, H); 256 threads; K walked in tiles of 64 channels.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gla_fwd_intra_kernel(const flab_args a) {
  constexpr int LD = GT + 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float *sQ = reinterpret_cast<float *>(smem_raw), *sK = sQ + C * LD, *sB = sK + C * LD;
  const int tid = threadIdx.x;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0);
  const size_t ks = tok_stride(a, a.K), offk = tok_off(a, s, hd, t0, a.K);
  const T *q = reinterpret_cast<const T *>(a.q) + offk, *k = reinterpret_cast<const T *>(a.k) + offk;
  const float *b = reinterpret_cast<const float *>(a.gk) + offk;
  // thread owns pairs p = tid, tid + 256, ... of the 64 x 64 grid (row-major); 16 pairs each
  float acc[16];
#pragma unroll
  for (int p = 0; p < 16; ++p) acc[p] = 0.f;
  for (int k0 = 0; k0 < a.K; k0 += GT) {
    const int kw = min(GT, a.K - k0);
    __syncthreads();
    for (int e = tid; e < C * GT; e += 256) {
      int r = e / GT, c = e - r * GT;
      bool ok = r < rows && c < kw;
      sQ[r * LD + c] = ok ? Num<T>::f(q[(size_t)r * ks + k0 + c]) : 0.f;
      sK[r * LD + c] = ok ? Num<T>::f(k[(size_t)r * ks + k0 + c]) : 0.f;
      sB[r * LD + c] = ok ? b[(size_t)r * ks + k0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 16; ++p) {
      const int e = tid + p * 256, i = e >> 6, j = e & 63;
      if (i >= j && i < rows) {
        float x = 0.f;
        for (int c = 0; c < kw; ++c) x = fmaf(sQ[i * LD + c] * sK[j * LD + c], expf(sB[i * LD + c] - sB[j * LD + c]), x);
        acc[p] += x;
      }
    }
  }
  float *A = reinterpret_cast<float *>(a.a) + tok_off(a, s, hd, t0, C);
  const size_t as_ = tok_stride(a, C);
#pragma unroll
  for (int p = 0; p < 16; ++p) {
    const int e = tid + p * 256, i = e >> 6, j = e & 63;
    if (i < rows) A[(size_t)i * as_ + j] = (i >= j) ? acc[p] * a.scale : 0.f;
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
  {
    const float *A = reinterpret_cast<const float *>(a.a) + tok_off(a, s, hd, t0, C);
    for (int e = tid; e < C * C; e += 128) {
      int i = e >> 6, j = e & 63;
      sA[i * LDP + j] = Num<T>::t((i < rows && i >= j) ? A[(size_t)i * as_ + j] : 0.f);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  {
    const float *b = reinterpret_cast<const float *>(a.gk) + offk;
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
  {
    const float *A = reinterpret_cast<const float *>(a.a) + tok_off(a, s, hd, t0, C);
    for (int e = tid; e < C * C; e += 128) {
      int i = e >> 6, j = e & 63;
      sA[i * LDP + j] = Num<T>::t((i < rows && i >= j) ? A[(size_t)i * as_ + j] : 0.f);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  {
    const float *b = reinterpret_cast<const float *>(a.gk) + offk;
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
// dq, dk, dg.  grid (NT, H, K/64); 256 threads.  Phase 1: inter-chunk products on the tile GEMM
// (do h^T, v dh^T), results parked in fp32 shared memory.  Phase 2: intra-chunk terms evaluated
// directly; thread = (token row, 4-way interleaved channel slice).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gla_bwd_dqkg_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int VP = round_up(a.V, 16);
  const int LDV = VP + Num<T>::pad;
  constexpr int LD = GT + 1;
  float *sDQ = reinterpret_cast<float *>(smem_raw);  // [64][LD] inter dq -> total dq
  float *sDK = sDQ + C * LD;                         // [64][LD]
  float *sGK = sDK + C * LD;                         // [64] per-channel chunk term of dg
  unsigned char *region = reinterpret_cast<unsigned char *>(sGK + GT);
  // phase 1 view
  T *sDO = reinterpret_cast<T *>(region);  // [64][LDV]
  T *sVV = sDO + C * LDV;                  // [64][LDV]
  T *sH = sVV + C * LDV;                   // [64 channels][LDV]
  T *sDH = sH + GT * LDV;                  // [64 channels][LDV]
  // phase 2 view
  float *sQ = reinterpret_cast<float *>(region);  // [64][LD]
  float *sK = sQ + C * LD;
  float *sB = sK + C * LD;
  float *sDA = sB + C * LD;  // [64][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y, k0 = blockIdx.z * GT;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0), last = rows - 1, kw = min(GT, a.K - k0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), as_ = tok_stride(a, C);
  const size_t offk = tok_off(a, s, hd, t0, a.K) + k0, offv = tok_off(a, s, hd, t0, a.V);
  const float *b = reinterpret_cast<const float *>(a.gk) + offk;

  // ---- phase 1
  {
    const size_t hoff = ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + (size_t)k0 * a.V;
    tile_load<T>(sDO, LDV, reinterpret_cast<const T *>(a.d_o) + offv, vs, rows, C, a.V, VP, tid, 256);
    tile_load<T>(sVV, LDV, reinterpret_cast<const T *>(a.v) + offv, vs, rows, C, a.V, VP, tid, 256);
    tile_load<T>(sH, LDV, reinterpret_cast<const T *>(a.h) + hoff, (size_t)a.V, kw, GT, a.V, VP, tid, 256);
    tile_load<T>(sDH, LDV, reinterpret_cast<const T *>(a.dh) + hoff, (size_t)a.V, kw, GT, a.V, VP, tid, 256);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    const int rb = warp & 3, ch = warp >> 2, m0 = rb * 16, n0 = ch * 32;
    float dq[1][4][4], dk[1][4][4];
    acc_zero(dq);
    acc_zero(dk);
    WarpGemm<1, 4, false, false, T>::run(dq, sDO, LDV, m0, sH, LDV, n0, VP);
    WarpGemm<1, 4, false, false, T>::run(dk, sVV, LDV, m0, sDH, LDV, n0, VP);
    FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
      float e1 = 0.f, e2 = 0.f;
      if (row < rows && col < kw) {
        float bi = b[(size_t)row * ks + col];
        e1 = expf(bi) * a.scale;
        e2 = expf(b[(size_t)last * ks + col] - bi);
      }
      sDQ[row * LD + col] = dq[mi][ni][r] * e1;
      sDK[row * LD + col] = dk[mi][ni][r] * e2;
    }
    // per-channel sum_v h * dh
    if (tid < GT) {
      float x = 0.f;
      if (tid < kw) {
        for (int c = 0; c < a.V; ++c) x = fmaf(Num<T>::f(sH[tid * LDV + c]), Num<T>::f(sDH[tid * LDV + c]), x);
        x *= expf(b[(size_t)last * ks + tid]);
      }
      sGK[tid] = x;
    }
  }
  __syncthreads();
  // ---- phase 2
  {
    const T *q = reinterpret_cast<const T *>(a.q) + offk, *k = reinterpret_cast<const T *>(a.k) + offk;
    const float *dA = reinterpret_cast<const float *>(a.da) + tok_off(a, s, hd, t0, C);
    for (int e = tid; e < C * GT; e += 256) {
      int r = e / GT, c = e - r * GT;
      bool ok = r < rows && c < kw;
      sQ[r * LD + c] = ok ? Num<T>::f(q[(size_t)r * ks + c]) : 0.f;
      sK[r * LD + c] = ok ? Num<T>::f(k[(size_t)r * ks + c]) : 0.f;
      sB[r * LD + c] = ok ? b[(size_t)r * ks + c] : 0.f;
      sDA[r * LD + c] = (r < rows && c <= r) ? dA[(size_t)r * as_ + c] : 0.f;  // c indexes the 64 columns of dA here
    }
    __syncthreads();
    // sum_j dk_inter * k per channel (before the intra terms are added)
    if (tid < GT) {
      float x = 0.f;
      for (int j = 0; j < rows; ++j) x = fmaf(sDK[j * LD + tid], sK[j * LD + tid], x);
      sGK[tid] += x;
    }
    __syncthreads();
    const int i = tid >> 2, sl = tid & 3;
    float aq[GT / 4], ak[GT / 4], bi[GT / 4];
#pragma unroll
    for (int m = 0; m < GT / 4; ++m) {
      aq[m] = 0.f;
      ak[m] = 0.f;
      bi[m] = sB[i * LD + sl + 4 * m];
    }
    if (i < rows) {
      for (int j = 0; j <= i; ++j) {
        const float d = sDA[i * LD + j];
#pragma unroll
        for (int m = 0; m < GT / 4; ++m) {
          const int c = sl + 4 * m;
          aq[m] = fmaf(d * sK[j * LD + c], expf(bi[m] - sB[j * LD + c]), aq[m]);
        }
      }
      for (int i2 = i; i2 < rows; ++i2) {
        const float d = sDA[i2 * LD + i];
#pragma unroll
        for (int m = 0; m < GT / 4; ++m) {
          const int c = sl + 4 * m;
          ak[m] = fmaf(d * sQ[i2 * LD + c], expf(sB[i2 * LD + c] - bi[m]), ak[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < GT / 4; ++m) {
      const int c = sl + 4 * m;
      sDQ[i * LD + c] += aq[m];
      sDK[i * LD + c] += ak[m];
    }
    __syncthreads();
    // outputs; dg = reverse in-chunk cumsum of (q dq - k dk) + per-channel chunk term
    T *dq = reinterpret_cast<T *>(a.dq) + offk, *dk = reinterpret_cast<T *>(a.dk) + offk;
    for (int e = tid; e < rows * kw; e += 256) {
      int r = e / kw, c = e - r * kw;
      dq[(size_t)r * ks + c] = Num<T>::t(sDQ[r * LD + c]);
      dk[(size_t)r * ks + c] = Num<T>::t(sDK[r * LD + c]);
    }
    if (tid < kw) {
      float *dg = reinterpret_cast<float *>(a.dgk) + offk;
      float run = sGK[tid];
      for (int r = rows - 1; r >= 0; --r) {
        run += sQ[r * LD + tid] * sDQ[r * LD + tid] - sK[r * LD + tid] * sDK[r * LD + tid];
        dg[(size_t)r * ks + tid] = run;
      }
    }
  }
  (void)lane;
}

template <typename T, int BV> static size_t gla_o_smem(const flab_args *a, bool dav) {
  const int KP = round_up(a->K, 16), LDK = KP + Num<T>::pad, LDV = BV + Num<T>::pad, LDP = C + Num<T>::pad;
  size_t e = (size_t)C * LDK + (size_t)C * LDV * (dav ? 2 : 1) + (size_t)C * LDP + (size_t)KP * LDV;
  return e * sizeof(T);
}

template <typename T> static int launch_gla_fwd_intra(const flab_args *a, cudaStream_t stream) {
  size_t smem = (size_t)3 * C * (GT + 1) * sizeof(float);
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
  size_t p2 = (size_t)4 * C * (GT + 1) * sizeof(float);
  size_t smem = ((size_t)2 * C * (GT + 1) + GT) * sizeof(float) + (p1 > p2 ? p1 : p2);
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
