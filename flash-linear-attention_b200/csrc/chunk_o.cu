// Chunk-parallel kernels: intra-chunk output and the gradients that do not need a scan.
//   fwd_o    : o  = scale * [(q h) * e^{b_i} + tril(q k^T * e^{b_i-b_j}) v]      (fla/ops/common/chunk_o.py:23-101)
//   bwd_dv   : dv = (k dh) * e^{b_L-b_j} + triu(k q^T * e^{b_i-b_j}) * scale do  (fla/ops/common/chunk_o.py:289-364)
//   dv_local : second term of bwd_dv only                                         (fla/ops/common/chunk_o.py:379-441)
//   dqkwg    : dq, dk, dw, dg                                                     (fla/ops/common/chunk_o.py:118-273)
// One CTA per (chunk, head).  All operands of a chunk are staged in shared memory once; the 64x64
// score tile is rounded to the element type in shared memory between its two contractions.
#include <cstdlib>

#include "common.cuh"

namespace flab {

enum { MODE_O = 0, MODE_DV = 1, MODE_DV_LOCAL = 2 };

// ------------------------------------------------------------------------------------------------
// fwd_o / bwd_dv / dv_local.  grid = (NT, H, V/BV); 4 warps, each owns 16 token rows.
// ------------------------------------------------------------------------------------------------
template <typename T, int MODE, int BV>
__global__ void __launch_bounds__(128) chunk_o_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KP = round_up(a.K, 16);
  const int LDK = KP + Num<T>::pad;
  constexpr int LDV = BV + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  T *sX1 = reinterpret_cast<T *>(smem_raw);  // [64][LDK] rows of the score tile (q for o, k for dv)
  T *sX2 = sX1 + C * LDK;                    // [64][LDK] columns of the score tile
  T *sY = sX2 + C * LDK;                     // [64][LDV] v (o) or do (dv); reused to stage the result
  T *sP = sY + C * LDV;                      // [64][LDP] score tile
  T *sH = sP + C * LDP;                      // [KP][LDV] chunk state tile (not for dv_local)
  float *sG = reinterpret_cast<float *>(sH + (MODE == MODE_DV_LOCAL ? 0 : (size_t)KP * LDV));  // [64]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y, v0 = blockIdx.z * BV;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0), last = rows - 1;
  const int vw = min(BV, a.V - v0);
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V);
  const T *X1 = reinterpret_cast<const T *>(MODE == MODE_O ? a.q : a.k) + tok_off(a, s, hd, t0, a.K);
  const T *X2 = reinterpret_cast<const T *>(MODE == MODE_O ? a.k : a.q) + tok_off(a, s, hd, t0, a.K);
  const T *Y = reinterpret_cast<const T *>(MODE == MODE_O ? a.v : a.d_o) + tok_off(a, s, hd, t0, a.V) + v0;
  T *Out = reinterpret_cast<T *>(MODE == MODE_O ? a.o : a.dv) + tok_off(a, s, hd, t0, a.V) + v0;
  const bool use_g = a.g != nullptr;

  tile_load<T>(sX1, LDK, X1, ks, rows, C, a.K, KP, tid, 128);
  tile_load<T>(sX2, LDK, X2, ks, rows, C, a.K, KP, tid, 128);
  tile_load<T>(sY, LDV, Y, vs, rows, C, vw, BV, tid, 128);
  if (MODE != MODE_DV_LOCAL) {
    const T *Hs = reinterpret_cast<const T *>(MODE == MODE_O ? a.h : a.dh) +
                  ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + v0;
    tile_load<T>(sH, LDV, Hs, (size_t)a.V, a.K, KP, vw, BV, tid, 128);
  }
  if (tid < C) {
    float gv = 0.f;
    if (use_g && tid < rows) gv = reinterpret_cast<const float *>(a.g)[tok_off(a, s, hd, t0 + tid, 1)];
    sG[tid] = gv;
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int m0 = warp * 16;
  const int g8 = lane >> 2, t4 = lane & 3;
  // score tile
  {
    float sc[1][8][4];
    acc_zero(sc);
    WarpGemm<1, 8, false, false, T>::run(sc, sX1, LDK, m0, sX2, LDK, 0, KP);
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) {
      float x = sc[mi][ni][r];
      if (MODE == MODE_O) {
        x = (row >= col) ? (use_g ? x * safe_exp(sG[row] - sG[col]) : x) : 0.f;
      } else {
        x = (row <= col) ? (use_g ? x * safe_exp(sG[col] - sG[row]) * a.scale : x * a.scale) : 0.f;
      }
      sc[mi][ni][r] = x;
    }
    acc_to_smem<1, 8, T>(sc, sP, LDP, m0, 0);
  }
  __syncwarp();
  constexpr int NI = BV / 8;
  float acc[1][NI][4];
  acc_zero(acc);
  if (MODE != MODE_DV_LOCAL) {
    WarpGemm<1, NI, false, true, T>::run(acc, sX1, LDK, m0, sH, LDV, 0, KP);
    if (use_g) {
      float s_lo, s_hi;
      if (MODE == MODE_O) {
        s_lo = expf(sG[m0 + g8]);
        s_hi = expf(sG[m0 + g8 + 8]);
      } else {
        s_lo = safe_exp(sG[last] - sG[m0 + g8]);
        s_hi = safe_exp(sG[last] - sG[m0 + g8 + 8]);
      }
#pragma unroll
      for (int ni = 0; ni < NI; ++ni) {
        acc[0][ni][0] *= s_lo;
        acc[0][ni][1] *= s_lo;
        acc[0][ni][2] *= s_hi;
        acc[0][ni][3] *= s_hi;
      }
    }
  }
  WarpGemm<1, NI, false, true, T>::run(acc, sP, LDP, m0, sY, LDV, 0, C);
  if (MODE == MODE_O) {
#pragma unroll
    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[0][ni][r] *= a.scale;
  }
  __syncthreads();  // every warp is done reading sY
  acc_to_smem<1, NI, T>(acc, sY, LDV, m0, 0);
  __syncthreads();
  tile_store<T>(Out, vs, sY, LDV, rows, vw, tid, 128);
  (void)t4;
}

template <typename T, int MODE> static int launch_chunk_o(const flab_args *a, cudaStream_t stream, const char *name) {
  const int KP = round_up(a->K, 16);
  const int LDK = KP + Num<T>::pad;
  const bool big = a->V > 64;
  const int BV = big ? 128 : 64;
  const int LDV = BV + Num<T>::pad, LDP = C + Num<T>::pad;
  size_t smem = ((size_t)2 * C * LDK + (size_t)C * LDV + (size_t)C * LDP) * sizeof(T) + C * sizeof(float);
  if (MODE != MODE_DV_LOCAL) smem += (size_t)KP * LDV * sizeof(T);
  dim3 grid(a->NT, a->H, cdiv(a->V, BV));
  if (big) {
    auto kern = chunk_o_kernel<T, MODE, 128>;
    if (int e = set_smem(kern, smem)) return e;
    kern<<<grid, 128, smem, stream>>>(*a);
  } else {
    auto kern = chunk_o_kernel<T, MODE, 64>;
    if (int e = set_smem(kern, smem)) return e;
    kern<<<grid, 128, smem, stream>>>(*a);
  }
  return check_launch(name);
}

// ------------------------------------------------------------------------------------------------
// dqkwg.  grid = (NT, H); 8 warps: warp = (row block rb of 16 tokens, column half ch of a 64-wide
// K tile).  K is walked in tiles of 64 channels.  Per tile, phase 1 contracts do / v / dv over V
// against the h / dh tiles (inter-chunk terms); the q / k / w tiles are then fetched into the same
// buffers and phase 2 adds the intra-chunk terms (contraction over the 64 tokens against ds).
// Re-using the buffers keeps the CTA under half of the SM's shared memory, so two CTAs overlap
// each other's load and compute phases.
// ------------------------------------------------------------------------------------------------
constexpr int QB = 64;  // K tile

template <typename T, bool USE_DW, int VPT /* padded V known at compile time, or 0 */>
__global__ void __launch_bounds__(256, 2) chunk_dqkwg_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int VP = VPT > 0 ? VPT : round_up(a.V, 16);
  const int LDV = VP + Num<T>::pad;
  constexpr int LDK = QB + Num<T>::pad;
  constexpr int LDP = C + Num<T>::pad;
  constexpr int NT3 = USE_DW ? 3 : 2;
  T *sV = reinterpret_cast<T *>(smem_raw);  // [64][LDV]
  T *sDO = sV + C * LDV;                    // [64][LDV]
  T *sDV = sDO + C * LDV;                   // [64][LDV]   (USE_DW)
  T *sU = sDV + (USE_DW ? C * LDV : 0);     // union: phase 1 {h, dh}[64][LDV]; phase 2 {q, k, w}[64][LDK]
  const int usz = max(2 * QB * LDV, NT3 * C * LDK);
  T *sH = sU, *sDH = sU + QB * LDV;
  T *sQ = sU, *sK = sU + C * LDK, *sW = sU + 2 * C * LDK;
  T *sDS = sU + usz;                                     // [64][LDP]
  float *sG = reinterpret_cast<float *>(sDS + C * LDP);  // [64]
  float *sDG = sG + C;                                   // [64]
  float *sRed = sDG + C;                                 // [2]: sum(h*dh), sum(dk*k)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2;
  int n, it;
  chunk_of(a, blockIdx.x, n, it);
  const int hd = blockIdx.y;
  const Seq s = seq_of(a, n);
  const int t0 = it * C, rows = min(C, s.len - t0), last = rows - 1;
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V);
  const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V);
  const bool use_g = a.g != nullptr;
  const size_t hbase = ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V;

  tile_load<T>(sV, LDV, reinterpret_cast<const T *>(a.v) + offv, vs, rows, C, a.V, VP, tid, 256);
  tile_load<T>(sDO, LDV, reinterpret_cast<const T *>(a.d_o) + offv, vs, rows, C, a.V, VP, tid, 256);
  if (USE_DW) tile_load<T>(sDV, LDV, reinterpret_cast<const T *>(a.dv) + offv, vs, rows, C, a.V, VP, tid, 256);
  {
    const int kw0 = min(QB, a.K);
    tile_load<T>(sH, LDV, reinterpret_cast<const T *>(a.h) + hbase, (size_t)a.V, kw0, QB, a.V, VP, tid, 256);
    tile_load<T>(sDH, LDV, reinterpret_cast<const T *>(a.dh) + hbase, (size_t)a.V, kw0, QB, a.V, VP, tid, 256);
  }
  if (tid < C) {
    float gv = 0.f;
    if (use_g && tid < rows) gv = reinterpret_cast<const float *>(a.g)[tok_off(a, s, hd, t0 + tid, 1)];
    sG[tid] = gv;
    sDG[tid] = 0.f;
  }
  if (tid < 2) sRed[tid] = 0.f;
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int rb = warp & 3, ch = warp >> 2;
  const int m0 = rb * 16, n0 = ch * 32;
  // ds = do v^T, masked / decayed / scaled once; kept in fp32 registers and as T in shared memory
  float ds[1][4][4];
  acc_zero(ds);
  WarpGemm<1, 4, false, false, T>::run(ds, sDO, LDV, m0, sV, LDV, n0, VP);
  FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
    float x = ds[mi][ni][r];
    x = (row >= col) ? (use_g ? x * safe_fexp<T>(sG[row] - sG[col]) : x) * a.scale : 0.f;
    ds[mi][ni][r] = x;
  }
  acc_to_smem<1, 4, T>(ds, sDS, LDP, m0, n0);

  const float e_lo = use_g ? fexp<T>(sG[m0 + g8]) : 1.f, e_hi = use_g ? fexp<T>(sG[m0 + g8 + 8]) : 1.f;
  const float f_lo = use_g ? safe_fexp<T>(sG[last] - sG[m0 + g8]) : 1.f, f_hi = use_g ? safe_fexp<T>(sG[last] - sG[m0 + g8 + 8]) : 1.f;
  float dg_lo = 0.f, dg_hi = 0.f;  // per-row partial of dg for rows m0+g8 and m0+g8+8
  float hdh = 0.f, dkk = 0.f;

  const int nk = cdiv(a.K, QB);
  for (int kt = 0; kt < nk; ++kt) {
    const int k0 = kt * QB, kw = min(QB, a.K - k0);
    if (kt > 0) {
      __syncthreads();  // previous tile's staged outputs have been read
      tile_load<T>(sH, LDV, reinterpret_cast<const T *>(a.h) + hbase + (size_t)k0 * a.V, (size_t)a.V, kw, QB, a.V, VP, tid, 256);
      tile_load<T>(sDH, LDV, reinterpret_cast<const T *>(a.dh) + hbase + (size_t)k0 * a.V, (size_t)a.V, kw, QB, a.V, VP, tid, 256);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
    }
    // ---- phase 1: inter-chunk terms
    float dq[1][4][4], dk[1][4][4], dw[1][4][4];
    acc_zero(dq);
    acc_zero(dk);
    WarpGemm<1, 4, false, false, T>::run(dq, sDO, LDV, m0, sH, LDV, n0, VP);
    WarpGemm<1, 4, false, false, T>::run(dk, sV, LDV, m0, sDH, LDV, n0, VP);
    if (USE_DW) {
      acc_zero(dw);
      WarpGemm<1, 4, false, false, T>::run(dw, sDV, LDV, m0, sH, LDV, n0, VP);
    }
    if (use_g) hdh += tile_dot<T>(sH, sDH, LDV, kw, VP, tid, 256);
    __syncthreads();  // every warp is done with h / dh
    tile_load<T>(sQ, LDK, reinterpret_cast<const T *>(a.q) + offk + k0, ks, rows, C, kw, QB, tid, 256);
    tile_load<T>(sK, LDK, reinterpret_cast<const T *>(a.k) + offk + k0, ks, rows, C, kw, QB, tid, 256);
    if (USE_DW) tile_load<T>(sW, LDK, reinterpret_cast<const T *>(a.w) + offk + k0, ks, rows, C, kw, QB, tid, 256);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    // ---- phase 2: gates, dg contributions, intra-chunk terms
    if (USE_DW) {
      // dw = -(dv h^T) * e^{b_i}; dg_i -= <w_i, dw_i> (dw before the sign flip)
      FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
        float x = dw[mi][ni][r] * ((r >> 1) ? e_hi : e_lo);
        if (use_g) {
          float wv = Num<T>::f(sW[row * LDK + col]);
          if (r >> 1) dg_hi -= wv * x; else dg_lo -= wv * x;
        }
        dw[mi][ni][r] = -x;
      }
    }
    FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
      const bool hi = r >> 1;
      const float xq = dq[mi][ni][r] * (hi ? e_hi : e_lo) * a.scale;
      const float xk = dk[mi][ni][r] * (hi ? f_hi : f_lo);
      if (use_g) dkk += xk * Num<T>::f(sK[row * LDK + col]);
      dq[mi][ni][r] = xq;
      dk[mi][ni][r] = xk;
    }
    WarpGemm<1, 4, false, true, T>::run(dq, sDS, LDP, m0, sK, LDK, n0, C);
    WarpGemm<1, 4, true, true, T>::run(dk, sDS, LDP, m0, sQ, LDK, n0, C);
    if (use_g) {
      // dg_i += <q_i, dq_i> - <k_i, dk_i> over the finished rows. This holds the inter-chunk terms and, because
      // rowsum_i(ds * (q k^T)) = <q_i, (ds k)_i> and colsum_j(ds * (q k^T)) = <k_j, (ds^T q)_j>, the intra-chunk
      // terms of fla/ops/common/chunk_o.py:520-560 as well, without forming q k^T.
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int col = n0 + ni * 8 + 2 * (lane & 3);
        const int o_lo = (m0 + g8) * LDK + col, o_hi = (m0 + g8 + 8) * LDK + col;
        const float2 q_lo = ld_pair<T>(sQ + o_lo), q_hi = ld_pair<T>(sQ + o_hi);
        const float2 k_lo = ld_pair<T>(sK + o_lo), k_hi = ld_pair<T>(sK + o_hi);
        dg_lo += dq[0][ni][0] * q_lo.x + dq[0][ni][1] * q_lo.y - dk[0][ni][0] * k_lo.x - dk[0][ni][1] * k_lo.y;
        dg_hi += dq[0][ni][2] * q_hi.x + dq[0][ni][3] * q_hi.y - dk[0][ni][2] * k_hi.x - dk[0][ni][3] * k_hi.y;
      }
    }
    __syncthreads();  // all warps done reading q / k / w
    acc_to_smem<1, 4, T>(dq, sQ, LDK, m0, n0);
    acc_to_smem<1, 4, T>(dk, sK, LDK, m0, n0);
    if (USE_DW) acc_to_smem<1, 4, T>(dw, sW, LDK, m0, n0);
    __syncthreads();
    tile_store<T>(reinterpret_cast<T *>(a.dq) + offk + k0, ks, sQ, LDK, rows, kw, tid, 256);
    tile_store<T>(reinterpret_cast<T *>(a.dk) + offk + k0, ks, sK, LDK, rows, kw, tid, 256);
    if (USE_DW) tile_store<T>(reinterpret_cast<T *>(a.dw) + offk + k0, ks, sW, LDK, rows, kw, tid, 256);
  }
  if (use_g) {
    dg_lo += __shfl_xor_sync(0xffffffffu, dg_lo, 1);
    dg_lo += __shfl_xor_sync(0xffffffffu, dg_lo, 2);
    dg_hi += __shfl_xor_sync(0xffffffffu, dg_hi, 1);
    dg_hi += __shfl_xor_sync(0xffffffffu, dg_hi, 2);
    if ((lane & 3) == 0) {
      atomicAdd(&sDG[m0 + g8], dg_lo);
      atomicAdd(&sDG[m0 + g8 + 8], dg_hi);
    }
    hdh = warp_sum(hdh);
    dkk = warp_sum(dkk);
    if (lane == 0) {
      atomicAdd(&sRed[0], hdh);
      atomicAdd(&sRed[1], dkk);
    }
    __syncthreads();
    if (tid < rows) {
      float x = sDG[tid];
      if (tid >= last) x += sRed[0] * expf(sG[last]) + sRed[1];
      reinterpret_cast<float *>(a.dg)[tok_off(a, s, hd, t0 + tid, 1)] = x;
    }
  }
}

template <typename T, bool USE_DW> static int launch_dqkwg(const flab_args *a, cudaStream_t stream) {
  const int VP = round_up(a->V, 16);
  const int LDV = VP + Num<T>::pad, LDK = QB + Num<T>::pad, LDP = C + Num<T>::pad;
  const int nt3 = USE_DW ? 3 : 2;
  const size_t usz = (size_t)(2 * QB * LDV > nt3 * C * LDK ? 2 * QB * LDV : nt3 * C * LDK);
  size_t elems = (size_t)nt3 * C * LDV + usz + (size_t)C * LDP;
  size_t smem = elems * sizeof(T) + (2 * C + 4) * sizeof(float);
  dim3 grid(a->NT, a->H);
#define FLAB_LAUNCH_DQKWG(VPT)                                   \
  {                                                              \
    auto kern = chunk_dqkwg_kernel<T, USE_DW, VPT>;              \
    if (int e = set_smem(kern, smem)) return e;                  \
    kern<<<grid, 256, smem, stream>>>(*a);                       \
  }
  if (VP == 128) FLAB_LAUNCH_DQKWG(128) else if (VP == 64) FLAB_LAUNCH_DQKWG(64) else FLAB_LAUNCH_DQKWG(0)
#undef FLAB_LAUNCH_DQKWG
  return check_launch("chunk_bwd_dqkwg");
}

// tcgen05 / TMA kernels for the shapes they cover (tc_chunk_o.cu); 1 = handled, 0 = not applicable
template <int MODE> int tc_chunk_o_try(const flab_args *a, cudaStream_t stream, const char *name);
int tc_dqkwg_try(const flab_args *a, cudaStream_t stream);
static bool tc_enabled() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("FLA_B200_NO_TC");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace flab

extern "C" {

int flab_chunk_fwd_o(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->h && a->o, FLAB_E_BADARG, "chunk_fwd_o needs q, k, v, h and o");
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "chunk_fwd_o: K = %d > 256", a->K);
  if (tc_enabled()) {
    int r = tc_chunk_o_try<MODE_O>(a, (cudaStream_t)stream, "chunk_fwd_o(tc)");
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_chunk_o<T, MODE_O>(a, (cudaStream_t)stream, "chunk_fwd_o")));
  return FLAB_OK;
}

int flab_chunk_bwd_dv(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->d_o && a->dh && a->dv, FLAB_E_BADARG, "chunk_bwd_dv needs q, k, d_o, dh and dv");
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "chunk_bwd_dv: K = %d > 256", a->K);
  if (tc_enabled()) {
    int r = tc_chunk_o_try<MODE_DV>(a, (cudaStream_t)stream, "chunk_bwd_dv(tc)");
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_chunk_o<T, MODE_DV>(a, (cudaStream_t)stream, "chunk_bwd_dv")));
  return FLAB_OK;
}

int flab_chunk_bwd_dv_local(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->d_o && a->dv, FLAB_E_BADARG, "chunk_bwd_dv_local needs q, k, d_o and dv");
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "chunk_bwd_dv_local: K = %d > 256", a->K);
  if (tc_enabled()) {
    int r = tc_chunk_o_try<MODE_DV_LOCAL>(a, (cudaStream_t)stream, "chunk_bwd_dv_local(tc)");
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_chunk_o<T, MODE_DV_LOCAL>(a, (cudaStream_t)stream, "chunk_bwd_dv_local")));
  return FLAB_OK;
}

int flab_chunk_bwd_dqkwg(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->h && a->dh && a->d_o && a->dq && a->dk, FLAB_E_BADARG,
               "chunk_bwd_dqkwg needs q, k, v, h, dh, d_o, dq and dk");
  FLAB_REQUIRE(!a->g || a->dg, FLAB_E_BADARG, "chunk_bwd_dqkwg: g given but dg is NULL");
  FLAB_REQUIRE(a->V <= 256, FLAB_E_UNSUPPORTED, "chunk_bwd_dqkwg: V = %d > 256", a->V);
  const bool use_dw = a->w != nullptr;
  if (use_dw) FLAB_REQUIRE(a->dv && a->dw, FLAB_E_BADARG, "chunk_bwd_dqkwg: w given but dv or dw is NULL");
  if (tc_enabled()) {
    const int r = tc_dqkwg_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  if (use_dw) {
    FLAB_DISPATCH_16(a->dtype, T, return (launch_dqkwg<T, true>(a, (cudaStream_t)stream)));
  } else {
    FLAB_DISPATCH_ALL(a->dtype, T, return (launch_dqkwg<T, false>(a, (cudaStream_t)stream)));
  }
  return FLAB_OK;
}
}
