// State recurrence of the (gated) delta rule: the serial part of the pipeline.
//   forward  (fla/ops/common/chunk_delta_h.py:27-119): per chunk
//       h[t] = S;  v_new = u - (w * e^{b}) bf(S);  S <- e^{b_L} S + (k * e^{b_L-b})^T bf(v_new)
//   backward (fla/ops/common/chunk_delta_h.py:136-237): per chunk, last to first
//       dh[t] = D; dv2 = dv + (k * e^{b_L-b}) bf(D);
//       D <- e^{b_L} D + (q*scale*e^{b})^T do - (w * e^{b})^T bf(dv2)
// One CTA (8 warps) owns all K rows and a 64-wide slab of V columns of one (sequence, head) state.
// The state stays in accumulator registers; its rounded copy goes through shared memory both as the
// operand of the dependent product and as the staging buffer of the coalesced h / dh store.
// The per-token gate factors are applied to the rows of the small [64 x 64] product / operand tiles
// (e^{b_i} (w S) instead of (e^{b_i} w) S, and k^T (e^{b_L-b_i} v_new) instead of (e^{b_L-b_i} k)^T v_new),
// so the [64 x K] token tiles are consumed exactly as cp.async delivered them and nothing but the two
// dependent products, two small conversions and four barriers sit on the serial path.
#include "common.cuh"

namespace flab {

constexpr int DBV = 64;  // V columns per slab (8 warps)

// NSLAB = 1: the CTA owns one 64-column slab of V.  NSLAB = 2: sixteen warps own two adjacent slabs
// and share the [tokens x K] tiles, so a K = V = 128 head is ONE CTA: with 128 (sequence, head) chains
// the whole scan is a single wave over the SMs instead of two.
template <typename T, int KP, bool BWD, int NSLAB>
__global__ void __launch_bounds__(256 * NSLAB) delta_h_kernel(const flab_args a) {
  constexpr int DTH = 256 * NSLAB;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LDK = KP + Num<T>::pad;
  constexpr int LDB = DBV + Num<T>::pad;
  // state tile KP x 64 over 8 warps
  constexpr int SR = KP >= 128 ? KP / 8 : 16;  // state rows per warp
  constexpr int SMI = SR / 16;
  constexpr int SNI = KP >= 128 ? 8 : 4;       // 64 or 32 columns per warp
  constexpr int NKT = BWD ? 3 : 2;  // [tokens x K] tiles per chunk: fwd (w, k); bwd (q, k, w)
  constexpr int NVT = BWD ? 2 : 1;  // [tokens x BV] tiles per chunk: fwd (u); bwd (do, dv)
  // Staggered buffering (backward, two slabs): k is needed only by the dependent product (c) and is kept in ONE
  // buffer that is refilled as soon as every warp has left (c); q and w, needed by the state update (e), stay
  // double-buffered. This is what lets two slabs fit in shared memory.
  constexpr bool STAG = BWD && NSLAB == 2;
  constexpr int NKBUF = STAG ? 5 : 2 * NKT;  // [tokens x K] tile buffers
  const int tid = threadIdx.x, slab = tid >> 8, stid = tid & 255, warp = stid >> 5;
  T *sKT = reinterpret_cast<T *>(smem_raw);        // [2][NKT][64][LDK] (staggered: k, then [2][q, w]); shared by the slabs
  T *sVTall = sKT + NKBUF * C * LDK;               // [NSLAB][2][NVT][64][LDB]
  T *sSall = sVTall + NSLAB * 2 * NVT * C * LDB;   // [NSLAB][KP][LDB] rounded state
  T *sOpall = sSall + NSLAB * KP * LDB;            // [NSLAB][64][LDB] gate-scaled operand of the state update
  float *sG = reinterpret_cast<float *>(sOpall + NSLAB * C * LDB);  // [2][64] gates; [64] e^{b}; [64] e^{b_L-b}
  float *sE1 = sG + 2 * C + slab * 2 * C, *sE2 = sE1 + C;  // per slab: the slabs only meet at barrier (1)
  T *sVT = sVTall + slab * 2 * NVT * C * LDB, *sS = sSall + slab * KP * LDB, *sOp = sOpall + slab * C * LDB;

  const int v0 = (blockIdx.x * NSLAB + slab) * DBV;
  const int n = blockIdx.y / a.H, hd = blockIdx.y % a.H;
  const Seq s = seq_of(a, n);
  const int vw = max(0, min(DBV, a.V - v0));
  const bool use_g = a.g != nullptr;
  const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V), gs = tok_stride(a, 1);
  const size_t offk = tok_off(a, s, hd, 0, a.K), offv = tok_off(a, s, hd, 0, a.V) + v0;
  const float *G = use_g ? reinterpret_cast<const float *>(a.g) + tok_off(a, s, hd, 0, 1) : nullptr;
  const T *kt_src[3];
  const T *vt_src[2];
  if (!BWD) {
    kt_src[0] = reinterpret_cast<const T *>(a.w) + offk;
    kt_src[1] = reinterpret_cast<const T *>(a.k) + offk;
    kt_src[2] = nullptr;
    vt_src[0] = reinterpret_cast<const T *>(a.u) + offv;
    vt_src[1] = nullptr;
  } else {
    kt_src[0] = reinterpret_cast<const T *>(a.q) + offk;
    kt_src[1] = reinterpret_cast<const T *>(a.k) + offk;
    kt_src[2] = reinterpret_cast<const T *>(a.w) + offk;
    vt_src[0] = reinterpret_cast<const T *>(a.d_o) + offv;
    vt_src[1] = reinterpret_cast<const T *>(a.dv) + offv;
  }
  T *Hout = reinterpret_cast<T *>(BWD ? a.dh : a.h);
  T *Vout = reinterpret_cast<T *>(BWD ? a.dv2 : a.v_new) + offv;
  const float *S0 = reinterpret_cast<const float *>(BWD ? a.dht : a.h0);
  float *S1 = reinterpret_cast<float *>(BWD ? a.dh0 : a.ht);

  float acc[SMI][SNI][4];
  acc_zero(acc);
  // warp tile of the state: rows [ms, ms + SR), columns [ns, ns + 8*SNI)
  const int ms = KP >= 128 ? warp * SR : (warp & 3) * 16;
  const int ns = KP >= 128 ? 0 : (warp >> 2) * 32;
  // warp tile of the [64 tokens x 64] product: rows [m0, m0+16), columns [n0, n0+32)
  const int m0 = (warp & 3) * 16, n0 = (warp >> 2) * 32;
  const size_t st_off = ((size_t)n * a.H + hd) * a.K * a.V;
  if (S0) {
    FLAB_ACC_FOREACH(SMI, SNI, ms, ns, row, col, mi, ni, r) {
      if (row < a.K && col < vw) acc[mi][ni][r] = S0[st_off + (size_t)row * a.V + v0 + col];
    }
  }

  // buffer of [tokens x K] tile j of the chunk held in stage `buf`
  auto ktile = [&](int j, int buf) -> T * {
    if (!STAG) return sKT + (buf * NKT + j) * C * LDK;
    return j == 1 ? sKT : sKT + (1 + buf * 2 + (j >> 1)) * C * LDK;
  };
  // tiles read by the dependent product (fwd: w, bwd: k), the [tokens x BV] tiles and the gates
  auto load_early = [&](int it, int buf) {
    const int t0 = it * C, rows = min(C, s.len - t0);
    constexpr int je = BWD ? 1 : 0;
    tile_load<T>(ktile(je, buf), LDK, kt_src[je] + (size_t)t0 * ks, ks, rows, C, a.K, KP, tid, DTH);
#pragma unroll
    for (int j = 0; j < NVT; ++j)
      tile_load<T>(sVT + (buf * NVT + j) * C * LDB, LDB, vt_src[j] + (size_t)t0 * vs, vs, rows, C, vw, DBV, stid, 256);
    cp_async_commit();
  };
  // tiles read by the state update (fwd: k, bwd: q and w)
  auto load_late = [&](int it, int buf) {
    const int t0 = it * C, rows = min(C, s.len - t0);
#pragma unroll
    for (int j = 0; j < NKT; ++j)
      if (j != (BWD ? 1 : 0))
        tile_load<T>(ktile(j, buf), LDK, kt_src[j] + (size_t)t0 * ks, ks, rows, C, a.K, KP, tid, DTH);
    cp_async_commit();
  };

  // gate of token `tid` of chunk `it`; fetched into a register one chunk ahead so that the load's latency is
  // never between two barriers of the serial chain
  auto gate_of = [&](int it) -> float {
    const int t0 = it * C;
    return (use_g && tid < C && t0 + tid < s.len) ? G[(size_t)(t0 + tid) * gs] : 0.f;
  };
  // barrier among the eight warps of one slab (everything between (1) and the next (1) is slab-private,
  // except the staggered k buffer, which is refilled after (3))
  auto slab_sync = [&]() {
    if (NSLAB == 1) __syncthreads();
    else asm volatile("bar.sync %0, 256;" ::"r"(1 + slab) : "memory");
  };
  const int first = BWD ? s.nt - 1 : 0, step = BWD ? -1 : 1;
  float g_pf = 0.f;
  if (s.nt > 0) {
    load_late(first, 0);
    load_early(first, 0);
    g_pf = gate_of(first);
  }
  for (int i = 0; i < s.nt; ++i) {
    const int it = first + i * step, cur = i & 1;
    if (tid < C) sG[cur * C + tid] = g_pf;
    cp_async_wait<0>();
    __syncthreads();  // (1) tiles of this chunk have landed; every warp is done with the previous chunk
    if (i + 1 < s.nt) {  // prefetch into the buffers the previous chunk used
      load_late(it + step, cur ^ 1);
      if (!STAG) load_early(it + step, cur ^ 1);
      g_pf = gate_of(it + step);
    }
    const int t0 = it * C, rows = min(C, s.len - t0), last = rows - 1;
    T *vt = sVT + cur * NVT * C * LDB;
    const float *gc = sG + cur * C;
    const float gl = gc[last];
    // (a) rounded state -> shared; per-token gate factors; bwd: do' = do * e^{b} * scale in place
    acc_to_smem<SMI, SNI, T>(acc, sS, LDB, ms, ns);
    if (stid < C) {
      sE1[stid] = use_g ? fexp<T>(gc[stid]) : 1.f;
      sE2[stid] = use_g ? fexp<T>(gl - gc[stid]) : 1.f;
    }
    if (BWD) {
      for (int e = stid; e < C * (DBV / 2); e += 256) {
        const int r_ = e / (DBV / 2), c_ = (e - r_ * (DBV / 2)) * 2;
        const float f = (use_g ? fexp<T>(gc[r_]) : 1.f) * a.scale;
        T *p = vt + r_ * LDB + c_;
        st_pair<T>(p, Num<T>::f(p[0]) * f, Num<T>::f(p[1]) * f);
      }
    }
    slab_sync();  // (2)
    // (b) state at the chunk boundary -> global (coalesced, off the critical path)
    {
      const size_t hoff = ((size_t)(s.c0 + it) * a.H + hd) * a.K * a.V + v0;
      tile_store<T>(Hout + hoff, (size_t)a.V, sS, LDB, a.K, vw, stid, 256);
    }
    // (c) the dependent product against the rounded state, gate applied to its rows
    {
      float p[1][4][4];
      acc_zero(p);
      const T *A = ktile(BWD ? 1 : 0, cur);  // bwd: k ; fwd: w
      WarpGemm<1, 4, false, true, T>::run(p, A, LDK, m0, sS, LDB, n0, KP);
      T *y = BWD ? vt + C * LDB : vt;  // bwd: dv ; fwd: u   (replaced in place by dv2 / v_new)
      float op[1][4][4];
      FLAB_ACC_FOREACH(1, 4, m0, n0, row, col, mi, ni, r) {
        const float base = Num<T>::f(y[row * LDB + col]);
        float x;
        if (!BWD) {
          x = rnd<T>(base - sE1[row] * p[mi][ni][r]);  // v_new
          op[mi][ni][r] = x * sE2[row];                // e^{b_L-b} v_new
        } else {
          x = rnd<T>(base + sE2[row] * p[mi][ni][r]);  // dv2
          op[mi][ni][r] = -x * sE1[row];               // -e^{b} dv2
        }
        p[mi][ni][r] = x;
      }
      acc_to_smem<1, 4, T>(p, y, LDB, m0, n0);
      acc_to_smem<1, 4, T>(op, sOp, LDB, m0, n0);
    }
    if (STAG) __syncthreads(); else slab_sync();  // (3)
    if (STAG && i + 1 < s.nt) load_early(it + step, cur ^ 1);  // every warp has left (c): the k buffer is free
    // (d) v_new / dv2 -> global
    tile_store<T>(Vout + (size_t)t0 * vs, vs, BWD ? vt + C * LDB : vt, LDB, rows, vw, stid, 256);
    // (e) state update
    if (use_g) {
      const float d = fexp<T>(gl);
#pragma unroll
      for (int mi = 0; mi < SMI; ++mi)
#pragma unroll
        for (int ni = 0; ni < SNI; ++ni)
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[mi][ni][r] *= d;
    }
    if (!BWD) {
      WarpGemm<SMI, SNI, true, true, T>::run(acc, ktile(1, cur), LDK, ms, sOp, LDB, ns, C);  // k^T (e^{b_L-b} v_new)
    } else {
      WarpGemm<SMI, SNI, true, true, T>::run(acc, ktile(0, cur), LDK, ms, vt, LDB, ns, C);              // q^T (scale e^{b} do)
      WarpGemm<SMI, SNI, true, true, T>::run(acc, ktile(2, cur), LDK, ms, sOp, LDB, ns, C);  // w^T (-e^{b} dv2)
    }
  }
  if (S1) {
    FLAB_ACC_FOREACH(SMI, SNI, ms, ns, row, col, mi, ni, r) {
      if (row < a.K && col < vw) S1[st_off + (size_t)row * a.V + v0 + col] = acc[mi][ni][r];
    }
  }
}

template <typename T, int KP, bool BWD, int NSLAB> static int launch_delta_h(const flab_args *a, cudaStream_t stream) {
  constexpr int LDK = KP + Num<T>::pad, LDB = DBV + Num<T>::pad;
  constexpr int NKT = BWD ? 3 : 2, NVT = BWD ? 2 : 1;
  constexpr int NKBUF = (BWD && NSLAB == 2) ? 5 : 2 * NKT;
  size_t smem = ((size_t)NKBUF * C * LDK + NSLAB * ((size_t)2 * NVT * C * LDB + (size_t)KP * LDB + (size_t)C * LDB)) * sizeof(T) +
                (2 + 2 * NSLAB) * C * sizeof(float);
  auto kern = delta_h_kernel<T, KP, BWD, NSLAB>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(cdiv(a->V, DBV * NSLAB), a->N * a->H), 256 * NSLAB, smem, stream>>>(*a);
  return check_launch(BWD ? "delta_bwd_dhu" : "delta_fwd_h");
}

template <bool BWD> static int dispatch_delta_h(const flab_args *a, void *stream) {
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "delta-rule state scan: K = %d > 256", a->K);
  // two slabs per CTA when V has at least two of them and the doubled per-slab buffers still fit (K <= 128)
  const bool two = a->K <= 128 && a->V > DBV;
  FLAB_DISPATCH_16(a->dtype, T, {
    if (a->K <= 64) return two ? (launch_delta_h<T, 64, BWD, 2>(a, (cudaStream_t)stream)) : (launch_delta_h<T, 64, BWD, 1>(a, (cudaStream_t)stream));
    if (a->K <= 128) return two ? (launch_delta_h<T, 128, BWD, 2>(a, (cudaStream_t)stream)) : (launch_delta_h<T, 128, BWD, 1>(a, (cudaStream_t)stream));
    return (launch_delta_h<T, 256, BWD, 1>(a, (cudaStream_t)stream));
  });
  return FLAB_OK;
}

// tcgen05 / TMA kernel for the shapes it covers (tc_delta_h.cu); 1 = handled, 0 = not applicable
int tc_delta_fwd_h_try(const flab_args *a, cudaStream_t stream);
int tc_delta_bwd_dhu_try(const flab_args *a, cudaStream_t stream);
static bool tc_scan_enabled() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("FLA_B200_NO_TC");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace flab

extern "C" {

int flab_delta_fwd_h(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  const bool state_only = (a->flags & FLAB_F_STATE_ONLY) != 0;
  FLAB_REQUIRE(a->k && a->w && a->u && (state_only || (a->h && a->v_new)), FLAB_E_BADARG, "delta_fwd_h needs k, w, u, h and v_new");
  FLAB_REQUIRE(!state_only || a->ht, FLAB_E_BADARG, "delta_fwd_h: a state-only scan needs ht");
  if (tc_scan_enabled()) {
    const int r = tc_delta_fwd_h_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_REQUIRE(!state_only, FLAB_E_UNSUPPORTED, "delta_fwd_h: state-only scans cover bf16 / fp16 with K = 128 and V a multiple of 64");
  return dispatch_delta_h<false>(a, stream);
}

int flab_delta_bwd_dhu(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  const bool state_only = (a->flags & FLAB_F_STATE_ONLY) != 0;
  FLAB_REQUIRE(a->q && a->k && a->w && a->d_o && a->dv && (state_only || (a->dh && a->dv2)), FLAB_E_BADARG,
               "delta_bwd_dhu needs q, k, w, d_o, dv, dh and dv2");
  FLAB_REQUIRE(!state_only || a->dh0, FLAB_E_BADARG, "delta_bwd_dhu: a state-only scan needs dh0");
  if (tc_scan_enabled()) {
    const int r = tc_delta_bwd_dhu_try(a, (cudaStream_t)stream);
    if (r != 0) return r < 0 ? r : FLAB_OK;
  }
  FLAB_REQUIRE(!state_only, FLAB_E_UNSUPPORTED, "delta_bwd_dhu: state-only scans cover bf16 / fp16 with K = 128 and V a multiple of 64");
  return dispatch_delta_h<true>(a, stream);
}
}
