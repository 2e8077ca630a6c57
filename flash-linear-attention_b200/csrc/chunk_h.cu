// Inter-chunk state recurrence for diagonal decay (scalar gate g, per-key-channel gate gk, per-value-channel
// gate gv, or none).
//   forward : h[t] = S;  S <- decay(S) + k~^T v~          (fla/ops/common/chunk_h.py:29-137)
//   backward: dh[t] = D; D <- decay(D) + q~^T do~         (fla/ops/common/chunk_h.py:156-271)
// gv decays the COLUMNS of the state (S <- S diag(e^{gv_L}), v~ = v e^{gv_L - gv}; backward do~ = do e^{gv}):
// the path the reference's GSA op takes (fla/ops/gsa/chunk.py:664-675); it may be combined with gk.
// One CTA owns a [64 x 64] tile of the [K x V] state of one (sequence, head) and walks the chunks
// serially; K and V tiles are independent, so the grid is (K/64, V/64, N*H).  The state tile lives
// in mma accumulator registers for the whole walk; k/v (q/do) tiles are double-buffered with cp.async.
#include "common.cuh"

namespace flab {

constexpr int HB = 64;  // state tile edge

template <typename T, int GATE /*0 none, 1 g, 2 gk*/, bool BWD, bool GV = false>
__global__ void __launch_bounds__(128) chunk_h_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LD = HB + Num<T>::pad;
  T *sX = reinterpret_cast<T *>(smem_raw);  // [2][64][LD]  k (fwd) or q (bwd) tile: rows = tokens
  T *sY = sX + 2 * C * LD;                  // [2][64][LD]  v (fwd) or do (bwd)
  T *sStage = sY + 2 * C * LD;              // [64][LD]     state tile staged for a coalesced store
  float *sG = reinterpret_cast<float *>(sStage + HB * LD);  // [2][64]
  float *sGK = sG + 2 * C;                                  // [2][64][HB+4] (GATE == 2 only)
  constexpr int LDG = HB + 4;
  float *sGV = sGK + (GATE == 2 ? 2 * C * LDG : 0);         // [2][64][HB+4] (GV only)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k0 = blockIdx.x * HB, v0 = blockIdx.y * HB;
  const int n = blockIdx.z / a.H, hd = blockIdx.z % a.H;
  const Seq s = seq_of(a, n);
  const int kw = min(HB, a.K - k0), vw = min(HB, a.V - v0);

  const T *X = reinterpret_cast<const T *>(BWD ? a.q : a.k) + tok_off(a, s, hd, 0, a.K) + k0;
  const T *Y = reinterpret_cast<const T *>(BWD ? a.d_o : a.v) + tok_off(a, s, hd, 0, a.V) + v0;
  const size_t xs = tok_stride(a, a.K), ys = tok_stride(a, a.V);
  const float *G = GATE == 1 ? reinterpret_cast<const float *>(a.g) + tok_off(a, s, hd, 0, 1) : nullptr;
  const size_t gs = tok_stride(a, 1);
  const float *GK = GATE == 2 ? reinterpret_cast<const float *>(a.gk) + tok_off(a, s, hd, 0, a.K) + k0 : nullptr;
  const float *GVp = GV ? reinterpret_cast<const float *>(a.gv) + tok_off(a, s, hd, 0, a.V) + v0 : nullptr;
  T *Hout = reinterpret_cast<T *>(BWD ? a.dh : a.h);
  const float *S0 = reinterpret_cast<const float *>(BWD ? a.dht : a.h0);
  float *S1 = reinterpret_cast<float *>(BWD ? a.dh0 : a.ht);

  float acc[1][8][4];
  acc_zero(acc);
  const int m0 = warp * 16;
  const size_t st_off = ((size_t)n * a.H + hd) * a.K * a.V;
  if (S0) {
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) {
      if (row < kw && col < vw) acc[mi][ni][r] = S0[st_off + (size_t)(k0 + row) * a.V + v0 + col];
    }
  }

  auto load = [&](int it, int buf) {
    const int t0 = it * C;
    const int rows = min(C, s.len - t0);
    tile_load<T>(sX + buf * C * LD, LD, X + (size_t)t0 * xs, xs, rows, C, kw, HB, tid, 128);
    tile_load<T>(sY + buf * C * LD, LD, Y + (size_t)t0 * ys, ys, rows, C, vw, HB, tid, 128);
    if (GATE == 2) tile_load<float>(sGK + buf * C * LDG, LDG, GK + (size_t)t0 * xs, xs, rows, C, kw, HB, tid, 128);
    if (GV) tile_load<float>(sGV + buf * C * LDG, LDG, GVp + (size_t)t0 * ys, ys, rows, C, vw, HB, tid, 128);
    cp_async_commit();
  };

  // scalar gate of token `tid` of chunk `it`, fetched into a register one chunk ahead: the load's latency never
  // sits between two barriers of the serial chain
  auto gate_of = [&](int it) -> float {
    const int t0 = it * C;
    return (GATE == 1 && tid < C && t0 + tid < s.len) ? G[(size_t)(t0 + tid) * gs] : 0.f;
  };
  const int first = BWD ? s.nt - 1 : 0, step = BWD ? -1 : 1;
  float g_pf = 0.f;
  if (s.nt > 0) {
    load(first, 0);
    g_pf = gate_of(first);
  }
  for (int i = 0; i < s.nt; ++i) {
    const int it = first + i * step, cur = i & 1;
    if (GATE == 1 && tid < C) sG[cur * C + tid] = g_pf;
    cp_async_wait<0>();
    __syncthreads();  // tiles of this chunk have landed; every warp is done with the previous chunk
    if (i + 1 < s.nt) {
      load(it + step, cur ^ 1);
      g_pf = gate_of(it + step);
    }
    T *x = sX + cur * C * LD, *y = sY + cur * C * LD;
    const int rows = min(C, s.len - it * C);
    const int last = rows - 1;
    // stage the state at the chunk boundary for the store
    acc_to_smem<1, 8, T>(acc, sStage, LD, m0, 0);
    // operand pre-scaling in shared memory (rounded to the element type like the reference does);
    // scalar gate: thread = (token row, half of the 64 columns), one exp per thread
    if (!BWD) {
      if (GATE == 1) {
        const int r_ = tid >> 1, c0 = (tid & 1) * (HB / 2);
        const float f = expf(sG[cur * C + last] - sG[cur * C + r_]);
#pragma unroll 4
        for (int c_ = c0; c_ < c0 + HB / 2; c_ += 2) {
          T *p = y + r_ * LD + c_;
          st_pair<T>(p, Num<T>::f(p[0]) * f, Num<T>::f(p[1]) * f);
        }
      } else if (GATE == 2) {
        const float *gk = sGK + cur * C * LDG;
        for (int e = tid; e < C * HB; e += 128) {
          int r_ = e / HB, c_ = e - r_ * HB;
          x[r_ * LD + c_] = Num<T>::t(Num<T>::f(x[r_ * LD + c_]) * expf(gk[last * LDG + c_] - gk[r_ * LDG + c_]));
        }
      }
    } else {
      if (GATE == 2) {
        const float *gk = sGK + cur * C * LDG;
        for (int e = tid; e < C * HB; e += 128) {
          int r_ = e / HB, c_ = e - r_ * HB;
          float qv = rnd<T>(Num<T>::f(x[r_ * LD + c_]) * a.scale) * expf(gk[r_ * LDG + c_]);
          x[r_ * LD + c_] = Num<T>::t(qv);
        }
      } else {
        const int r_ = tid >> 1, c0 = (tid & 1) * (HB / 2);
        const float f = GATE == 1 ? expf(sG[cur * C + r_]) : 1.f;
#pragma unroll 4
        for (int c_ = c0; c_ < c0 + HB / 2; c_ += 2) {
          T *p = x + r_ * LD + c_;
          st_pair<T>(p, rnd<T>(Num<T>::f(p[0]) * a.scale) * f, rnd<T>(Num<T>::f(p[1]) * a.scale) * f);
        }
      }
    }
    if (GV) {
      // value-channel gate: forward v~ = v e^{gv_L - gv}, backward do~ = do e^{gv}; rounded to the element type
      const float *gv = sGV + cur * C * LDG;
      for (int e = tid; e < C * HB; e += 128) {
        int r_ = e / HB, c_ = e - r_ * HB;
        const float f = BWD ? expf(gv[r_ * LDG + c_]) : expf(gv[last * LDG + c_] - gv[r_ * LDG + c_]);
        y[r_ * LD + c_] = Num<T>::t(Num<T>::f(y[r_ * LD + c_]) * f);
      }
    }
    __syncthreads();
    {
      const size_t hoff = ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + (size_t)k0 * a.V + v0;
      tile_store<T>(Hout + hoff, (size_t)a.V, sStage, LD, kw, vw, tid, 128);
    }
    // decay the running state
    if (GATE == 1) {
      const float d = expf(sG[cur * C + last]);
#pragma unroll
      for (int ni = 0; ni < 8; ++ni)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[0][ni][r] *= d;
    } else if (GATE == 2) {
      const float *gk = sGK + cur * C * LDG + last * LDG;
      const float d_lo = expf(gk[m0 + (lane >> 2)]), d_hi = expf(gk[m0 + (lane >> 2) + 8]);
#pragma unroll
      for (int ni = 0; ni < 8; ++ni) {
        acc[0][ni][0] *= d_lo;
        acc[0][ni][1] *= d_lo;
        acc[0][ni][2] *= d_hi;
        acc[0][ni][3] *= d_hi;
      }
    }
    if (GV) {
      const float *gv = sGV + cur * C * LDG + last * LDG;
#pragma unroll
      for (int ni = 0; ni < 8; ++ni) {
        const float d0 = expf(gv[8 * ni + 2 * (lane & 3)]), d1 = expf(gv[8 * ni + 2 * (lane & 3) + 1]);
        acc[0][ni][0] *= d0;
        acc[0][ni][1] *= d1;
        acc[0][ni][2] *= d0;
        acc[0][ni][3] *= d1;
      }
    }
    WarpGemm<1, 8, true, true, T>::run(acc, x, LD, m0, y, LD, 0, C);
  }
  if (S1) {
    FLAB_ACC_FOREACH(1, 8, m0, 0, row, col, mi, ni, r) {
      if (row < kw && col < vw) S1[st_off + (size_t)(k0 + row) * a.V + v0 + col] = acc[mi][ni][r];
    }
  }
}

template <typename T, bool BWD> static int launch_chunk_h(const flab_args *a, cudaStream_t stream) {
  constexpr int LD = HB + Num<T>::pad;
  const int gate = a->gk ? 2 : (a->g ? 1 : 0);
  size_t smem = (size_t)(5 * C * LD) * sizeof(T) + 2 * C * sizeof(float);
  if (gate == 2) smem += (size_t)2 * C * (HB + 4) * sizeof(float);
  if (a->gv) smem += (size_t)2 * C * (HB + 4) * sizeof(float);
  dim3 grid(cdiv(a->K, HB), cdiv(a->V, HB), a->N * a->H);
#define FLAB_LAUNCH_H(G, GVF)                                     \
  {                                                               \
    auto kern = chunk_h_kernel<T, G, BWD, GVF>;                   \
    if (int e = set_smem(kern, smem)) return e;                   \
    kern<<<grid, 128, smem, stream>>>(*a);                        \
  }
  if (a->gv) {
    if (gate == 0) FLAB_LAUNCH_H(0, true) else FLAB_LAUNCH_H(2, true)
  } else {
    if (gate == 0) FLAB_LAUNCH_H(0, false) else if (gate == 1) FLAB_LAUNCH_H(1, false) else FLAB_LAUNCH_H(2, false)
  }
#undef FLAB_LAUNCH_H
  return check_launch(BWD ? "chunk_bwd_dh" : "chunk_fwd_h");
}

// tcgen05 / TMA kernels for the shapes they cover (tc_delta_h.cu); 1 = handled, 0 = not applicable
int tc_chunk_fwd_h_try(const flab_args *a, cudaStream_t stream);
int tc_chunk_bwd_dh_try(const flab_args *a, cudaStream_t stream);
static bool tc_scan_on() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("FLA_B200_NO_TC");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace flab

extern "C" {

int flab_chunk_fwd_h(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->k && a->v && a->h, FLAB_E_BADARG, "chunk_fwd_h needs k, v and h");
  FLAB_REQUIRE(!(a->g && a->gk), FLAB_E_UNSUPPORTED, "chunk_fwd_h: g and gk together are not supported");
  FLAB_REQUIRE(!(a->g && a->gv), FLAB_E_UNSUPPORTED, "chunk_fwd_h: g and gv together are not supported");
  if (tc_scan_on()) {
    const int r = tc_chunk_fwd_h_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_chunk_h<T, false>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_chunk_bwd_dh(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->d_o && a->dh, FLAB_E_BADARG, "chunk_bwd_dh needs q, d_o and dh");
  FLAB_REQUIRE(!(a->g && a->gk), FLAB_E_UNSUPPORTED, "chunk_bwd_dh: g and gk together are not supported");
  FLAB_REQUIRE(!(a->g && a->gv), FLAB_E_UNSUPPORTED, "chunk_bwd_dh: g and gv together are not supported");
  if (tc_scan_on()) {
    const int r = tc_chunk_bwd_dh_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_chunk_h<T, true>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}
}
