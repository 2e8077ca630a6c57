// Token-recurrent kernels (decode and the reference's test oracles).
//
// Forward: one thread owns one value column of the [K x V] state and keeps its K entries in
// registers, so the per-token reductions over K (o = S^T q, the delta-rule correction S^T k) are
// thread-local; a warp reads 32 adjacent columns, i.e. one 128-byte row segment of the fp32 state
// per load.  The state is read once and written once per call - decode (T = 1) is a pure stream
// over the state and runs at HBM speed.
//   generic gates g / gk / gv:  fla/ops/common/fused_recurrent.py:27-128
//   delta rule (optional scalar gate): fla/ops/delta_rule/fused_recurrent.py:19-109,
//                                      fla/ops/gated_delta_rule/fused_recurrent.py:19-110
// Backward (training-time check path): the state lives in shared memory and every token does row
// and column reductions over it (fla/ops/common/fused_recurrent.py:145-319,
// fla/ops/delta_rule/fused_recurrent.py:118-290).
#include "common.cuh"

namespace flab {

constexpr int RC_COLS = 32;  // value columns per CTA in the forward kernels (one warp wide)

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
template <typename T, int KPT, bool DELTA>
__global__ void __launch_bounds__(RC_COLS * 2) recurrent_fwd_kernel(const flab_args a) {
  // blockDim = (32, KG): KG groups split K when K > KPT
  __shared__ float sQ[256], sK[256], sE[256];  // q*scale, k, exp(gk) of the current token
  __shared__ float sRed[2][2][RC_COLS];        // cross-group partial sums
  const int KG = blockDim.y, kg = threadIdx.y, lane = threadIdx.x;
  const int tid = kg * RC_COLS + lane, nthr = RC_COLS * KG;
  const int n = blockIdx.y / a.H, hd = blockIdx.y % a.H;
  const Seq s = seq_of(a, n);
  const int col = blockIdx.x * RC_COLS + lane;
  const bool cok = col < a.V;
  const int kbase = kg * KPT;
  const int K = a.K, V = a.V;
  const bool rev = (a.flags & FLAB_F_REVERSE) != 0;
  const bool beta_vec = (a.flags & FLAB_F_BETA_VECTOR) != 0;

  float S[KPT];
  const size_t st_off = ((size_t)n * a.H + hd) * K * V;
  const float *h0 = reinterpret_cast<const float *>(a.h0);
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    int kk = kbase + i;
    S[i] = (h0 && cok && kk < K) ? h0[st_off + (size_t)kk * V + col] : 0.f;
  }
  const T *q = reinterpret_cast<const T *>(a.q), *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v);
  const float *g = reinterpret_cast<const float *>(a.g), *gk = reinterpret_cast<const float *>(a.gk),
              *gv = reinterpret_cast<const float *>(a.gv);
  const T *beta = reinterpret_cast<const T *>(a.beta);

  for (int i_t = 0; i_t < s.len; ++i_t) {
    const int t = rev ? s.len - 1 - i_t : i_t;
    const size_t ok_ = tok_off(a, s, hd, t, K), ov = tok_off(a, s, hd, t, V), o1 = tok_off(a, s, hd, t, 1);
    __syncthreads();
    for (int i = tid; i < K; i += nthr) {
      sQ[i] = Num<T>::f(q[ok_ + i]) * a.scale;
      sK[i] = Num<T>::f(k[ok_ + i]);
      if (gk) sE[i] = expf(gk[ok_ + i]);
    }
    __syncthreads();
    float vv = cok ? Num<T>::f(v[ov + col]) : 0.f;
    float dec = 1.f;
    if (g) dec = expf(g[o1]);
    if (gv && cok) dec *= expf(gv[ov + col]);
    float o_acc = 0.f;
    if (!DELTA) {
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        int kk = kbase + i;
        if (kk < K) {
          float e = gk ? dec * sE[kk] : dec;
          S[i] = S[i] * e + sK[kk] * vv;
          o_acc = fmaf(S[i], sQ[kk], o_acc);
        }
      }
    } else {
      float p = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        int kk = kbase + i;
        if (kk < K) {
          S[i] *= dec;
          p = fmaf(S[i], sK[kk], p);
        }
      }
      if (KG > 1) {
        sRed[0][kg][lane] = p;
        __syncthreads();
        p = sRed[0][0][lane] + sRed[0][1][lane];
      }
      float u_ = vv - p;
      if (a.u && cok && kg == 0) reinterpret_cast<T *>(a.u)[ov + col] = Num<T>::t(u_);
      float b = 1.f;
      if (beta) b = beta_vec ? (cok ? Num<T>::f(beta[ov + col]) : 0.f) : Num<T>::f(beta[o1]);
      float vn = u_ * b;
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        int kk = kbase + i;
        if (kk < K) {
          S[i] = fmaf(sK[kk], vn, S[i]);
          o_acc = fmaf(S[i], sQ[kk], o_acc);
        }
      }
    }
    if (KG > 1) {
      sRed[1][kg][lane] = o_acc;
      __syncthreads();
      o_acc = sRed[1][0][lane] + sRed[1][1][lane];
    }
    if (cok && kg == 0) {
      if (DELTA) reinterpret_cast<T *>(a.o)[ov + col] = Num<T>::t(o_acc);
      else reinterpret_cast<float *>(a.o)[ov + col] = o_acc;
    }
  }
  float *ht = reinterpret_cast<float *>(a.ht);
  if (ht && cok) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
      int kk = kbase + i;
      if (kk < K) ht[st_off + (size_t)kk * V + col] = S[i];
    }
  }
}

template <typename T, bool DELTA> static int launch_recurrent_fwd(const flab_args *a, cudaStream_t stream) {
  dim3 grid(cdiv(a->V, RC_COLS), a->N * a->H);
  if (a->K <= 64) {
    recurrent_fwd_kernel<T, 64, DELTA><<<grid, dim3(RC_COLS, 1), 0, stream>>>(*a);
  } else if (a->K <= 128) {
    recurrent_fwd_kernel<T, 128, DELTA><<<grid, dim3(RC_COLS, 1), 0, stream>>>(*a);
  } else {
    recurrent_fwd_kernel<T, 128, DELTA><<<grid, dim3(RC_COLS, 2), 0, stream>>>(*a);
  }
  return check_launch(DELTA ? "recurrent_delta_fwd" : "recurrent_fwd");
}

// ------------------------------------------------------------------------------------------------
// backward: state in shared memory, 256 threads; rows = key channels, columns = value channels
// ------------------------------------------------------------------------------------------------
template <typename T, bool DELTA>
__global__ void __launch_bounds__(256) recurrent_bwd_kernel(const flab_args a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int K = a.K, V = a.V, VS = V | 1;  // odd row stride: conflict-free row walks
  float *S = reinterpret_cast<float *>(smem_raw);  // [K][VS]
  float *sq = S + (size_t)K * VS, *sk = sq + K, *sek = sk + K, *sdk = sek + K;  // [K] each
  float *sv = sdk + K, *sdo = sv + V, *sev = sdo + V, *sdv = sev + V;           // [V] each
  __shared__ float sScal[2];
  const int tid = threadIdx.x;
  const int n = blockIdx.x / a.H, hd = blockIdx.x % a.H;
  const Seq s = seq_of(a, n);
  const bool rev = (a.flags & FLAB_F_REVERSE) != 0;
  const bool beta_vec = (a.flags & FLAB_F_BETA_VECTOR) != 0;
  const T *q = reinterpret_cast<const T *>(a.q), *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v),
          *d_o = reinterpret_cast<const T *>(a.d_o), *beta = reinterpret_cast<const T *>(a.beta);
  const float *g = reinterpret_cast<const float *>(a.g), *gk = reinterpret_cast<const float *>(a.gk),
              *gv = reinterpret_cast<const float *>(a.gv);
  float *dq = reinterpret_cast<float *>(a.dq), *dk = reinterpret_cast<float *>(a.dk), *dv = reinterpret_cast<float *>(a.dv);
  float *dbeta = reinterpret_cast<float *>(a.dbeta);
  const size_t st_off = ((size_t)n * a.H + hd) * K * V;
  const float *h0 = reinterpret_cast<const float *>(a.h0), *dht = reinterpret_cast<const float *>(a.dht);
  float *dh0 = reinterpret_cast<float *>(a.dh0);

  auto fill_state = [&](const float *src) {
    for (int e = tid; e < K * V; e += 256) {
      int r = e / V, c = e - r * V;
      S[r * VS + c] = src ? src[st_off + e] : 0.f;
    }
  };
  auto load_tok = [&](int t) {
    const size_t ok_ = tok_off(a, s, hd, t, K), ov = tok_off(a, s, hd, t, V), o1 = tok_off(a, s, hd, t, 1);
    for (int i = tid; i < K; i += 256) {
      sq[i] = Num<T>::f(q[ok_ + i]) * a.scale;
      sk[i] = Num<T>::f(k[ok_ + i]);
      sek[i] = gk ? expf(gk[ok_ + i]) : 1.f;
    }
    const float eg = g ? expf(g[o1]) : 1.f;
    for (int i = tid; i < V; i += 256) {
      float b = 1.f;
      if (DELTA && beta) b = beta_vec ? Num<T>::f(beta[ov + i]) : Num<T>::f(beta[o1]);
      sv[i] = Num<T>::f(v[ov + i]);
      sdo[i] = Num<T>::f(d_o[ov + i]);
      sev[i] = DELTA ? b : (gv ? expf(gv[ov + i]) * eg : eg);  // delta: beta; generic: column decay incl. g
    }
  };

  if (!DELTA) {
    // pass 1: rebuild the states in processing order; dq_t = scale * h_t do_t
    fill_state(h0);
    for (int i_t = 0; i_t < s.len; ++i_t) {
      const int t = rev ? s.len - 1 - i_t : i_t;
      __syncthreads();
      load_tok(t);
      __syncthreads();
      for (int e = tid; e < K * V; e += 256) {
        int r = e / V, c = e - r * V;
        S[r * VS + c] = S[r * VS + c] * sek[r] * sev[c] + sk[r] * sv[c];
      }
      __syncthreads();
      const size_t ok_ = tok_off(a, s, hd, t, K);
      for (int r = tid; r < K; r += 256) {
        float acc = 0.f;
        for (int c = 0; c < V; ++c) acc = fmaf(S[r * VS + c], sdo[c], acc);
        dq[ok_ + r] = acc * a.scale;
      }
    }
    // pass 2: opposite order
    __syncthreads();
    fill_state(dht);
    for (int i_t = 0; i_t < s.len; ++i_t) {
      const int t = rev ? i_t : s.len - 1 - i_t;
      __syncthreads();
      load_tok(t);
      __syncthreads();
      for (int e = tid; e < K * V; e += 256) {
        int r = e / V, c = e - r * V;
        S[r * VS + c] += sq[r] * sdo[c];
      }
      __syncthreads();
      const size_t ok_ = tok_off(a, s, hd, t, K), ov = tok_off(a, s, hd, t, V);
      for (int r = tid; r < K; r += 256) {
        float acc = 0.f;
        for (int c = 0; c < V; ++c) acc = fmaf(S[r * VS + c], sv[c], acc);
        dk[ok_ + r] = acc;
      }
      for (int c = tid; c < V; c += 256) {
        float acc = 0.f;
        for (int r = 0; r < K; ++r) acc = fmaf(S[r * VS + c], sk[r], acc);
        dv[ov + c] = acc;
      }
      __syncthreads();
      for (int e = tid; e < K * V; e += 256) {
        int r = e / V, c = e - r * V;
        S[r * VS + c] *= sek[r] * sev[c];
      }
    }
    __syncthreads();
    if (dh0)
      for (int e = tid; e < K * V; e += 256) dh0[st_off + e] = S[(e / V) * VS + (e % V)];
  } else {
    // pass 1 (last token to first): dk, dv, dbeta with the running state gradient
    fill_state(dht);
    for (int t = s.len - 1; t >= 0; --t) {
      __syncthreads();
      load_tok(t);
      if (tid == 0) sScal[0] = 0.f;
      __syncthreads();
      for (int e = tid; e < K * V; e += 256) {
        int r = e / V, c = e - r * V;
        S[r * VS + c] += sq[r] * sdo[c];
      }
      __syncthreads();
      const size_t ok_ = tok_off(a, s, hd, t, K), ov = tok_off(a, s, hd, t, V), o1 = tok_off(a, s, hd, t, 1);
      for (int r = tid; r < K; r += 256) {
        float acc = 0.f;
        for (int c = 0; c < V; ++c) acc = fmaf(S[r * VS + c], sv[c] * sev[c], acc);
        dk[ok_ + r] = acc;
      }
      float db_part = 0.f;
      for (int c = tid; c < V; c += 256) {
        float acc = 0.f;
        for (int r = 0; r < K; ++r) acc = fmaf(S[r * VS + c], sk[r], acc);
        float db = acc * sv[c];
        if (beta_vec) dbeta[ov + c] = db; else db_part += db;
        acc *= sev[c];
        sdv[c] = acc;
        dv[ov + c] = acc;
      }
      if (!beta_vec) {
        db_part = warp_sum(db_part);
        if ((tid & 31) == 0) atomicAdd(&sScal[0], db_part);
      }
      __syncthreads();
      if (!beta_vec && tid == 0) dbeta[o1] = sScal[0];
      for (int e = tid; e < K * V; e += 256) {
        int r = e / V, c = e - r * V;
        S[r * VS + c] -= sk[r] * sdv[c];
      }
    }
    __syncthreads();
    if (dh0)
      for (int e = tid; e < K * V; e += 256) dh0[st_off + e] = S[(e / V) * VS + (e % V)];
    // pass 2 (first token to last): finish dk and compute dq with the forward state
    __syncthreads();
    fill_state(h0);
    for (int t = 0; t < s.len; ++t) {
      __syncthreads();
      load_tok(t);
      const size_t ok_ = tok_off(a, s, hd, t, K), ov = tok_off(a, s, hd, t, V);
      for (int c = tid; c < V; c += 256) sdv[c] = dv[ov + c];
      __syncthreads();
      for (int r = tid; r < K; r += 256) {
        float acc = 0.f;
        for (int c = 0; c < V; ++c) acc = fmaf(S[r * VS + c], sdv[c], acc);
        dk[ok_ + r] -= acc;
      }
      __syncthreads();
      for (int e = tid; e < K * V; e += 256) {
        int r = e / V, c = e - r * V;
        S[r * VS + c] += sk[r] * sv[c] * sev[c];
      }
      __syncthreads();
      for (int r = tid; r < K; r += 256) {
        float acc = 0.f;
        for (int c = 0; c < V; ++c) acc = fmaf(S[r * VS + c], sdo[c], acc);
        dq[ok_ + r] = acc * a.scale;
      }
    }
  }
}

template <typename T, bool DELTA> static int launch_recurrent_bwd(const flab_args *a, cudaStream_t stream) {
  const int VS = a->V | 1;
  size_t smem = ((size_t)a->K * VS + 4 * (size_t)a->K + 4 * (size_t)a->V) * sizeof(float);
  auto kern = recurrent_bwd_kernel<T, DELTA>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<a->N * a->H, 256, smem, stream>>>(*a);
  return check_launch(DELTA ? "recurrent_delta_bwd" : "recurrent_bwd");
}

}  // namespace flab

extern "C" {

int flab_recurrent_fwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->o, FLAB_E_BADARG, "recurrent_fwd needs q, k, v and o");
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "recurrent_fwd: K = %d > 256", a->K);
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_recurrent_fwd<T, false>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_recurrent_delta_fwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->o, FLAB_E_BADARG, "recurrent_delta_fwd needs q, k, v and o");
  FLAB_REQUIRE(!a->gk && !a->gv, FLAB_E_UNSUPPORTED, "recurrent_delta_fwd: only the scalar gate g is supported");
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "recurrent_delta_fwd: K = %d > 256", a->K);
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_recurrent_fwd<T, true>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_recurrent_bwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->d_o && a->dq && a->dk && a->dv, FLAB_E_BADARG,
               "recurrent_bwd needs q, k, v, d_o, dq, dk and dv");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_recurrent_bwd<T, false>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_recurrent_delta_bwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->d_o && a->dq && a->dk && a->dv && a->dbeta, FLAB_E_BADARG,
               "recurrent_delta_bwd needs q, k, v (the stored u), d_o, dq, dk, dv and dbeta");
  FLAB_REQUIRE(!a->g && !a->gk && !a->gv, FLAB_E_UNSUPPORTED, "recurrent_delta_bwd: gates are not supported");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_recurrent_bwd<T, true>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}
}
