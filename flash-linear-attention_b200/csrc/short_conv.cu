// Causal depthwise short convolution with optional SiLU, the per-layer convolution the reference's layers apply to q, k
// and v before the chunk op (fla/modules/convolution.py:79-216; fla/layers/gated_deltanet.py:205-228):
//   pre[b,t,d] = bias[d] + sum_{w<W} weight[d,w] x[b, t-(W-1)+w, d]   (x = 0 before the sequence),  y = silu(pre) or pre
//   decode step (:189-216): the cache [B, D, W] is shifted by one, x appended, y = act(bias + sum_w cache[., ., w] weight[., w])
// Layout [B, T, D] with the channels contiguous: a thread owns four channels and walks TT tokens with the last
// W-1 inputs in registers, so x is read once (plus a halo of W-1 tokens per tile) and y written once.
// Backward: pre is recomputed, dpre = dy * act'(pre);  dx[t] = sum_w weight[d,w] dpre[t+(W-1)-w];
// dweight[d,w] = sum_{b,t} dpre[t] x[t-(W-1)+w], dbias[d] = sum dpre: per-thread partial sums over the tile, then fp32
// atomics into [D, W] / [D] buffers the caller has zeroed.
#include <type_traits>

#include "common.cuh"

namespace flab {

constexpr int SC_TT = 32;    // tokens per thread
constexpr int SC_WMAX = 8;   // longest supported filter (decode step)
constexpr int SC_UN = 4;     // tokens whose loads are in flight together

// EV channels per thread: four in the forward kernel (8 bytes of a 16-bit type, 16 bytes of fp32), two in the backward
// kernel, whose register windows (inputs, dpre, dweight sums) otherwise leave two blocks per SM
template <typename T, int EV> struct __align__(EV * sizeof(T)) CV {
  static constexpr int N = EV;
  T v[N];
};
constexpr int SC_EVF = 4, SC_EVB = 2;

// sigmoid: tanh.approx for bf16, exponential + hardware reciprocal for fp16, exponential + IEEE division for fp32
template <typename T> __device__ __forceinline__ float sigm(float x) {
  if (std::is_same<T, bf16>::value) {  // one special-function instruction; its 5e-4 absolute error is below half a bf16 ulp of the product
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
  }
  return sizeof(T) == 2 ? __fdividef(1.f, 1.f + __expf(-x)) : 1.f / (1.f + __expf(-x));
}
template <typename T> __device__ __forceinline__ float silu_f(float x) { return x * sigm<T>(x); }
template <typename T> __device__ __forceinline__ float silu_grad_f(float x) {
  const float s = sigm<T>(x);
  return s * (1.f + x * (1.f - s));
}

// grid (ceil(T / TT), B, ceil(D / (EV * 256)))
template <typename T, int W, bool ACT, int EV>
__global__ void __launch_bounds__(256, 3) short_conv_fwd_kernel(const T *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                                                             T *__restrict__ y, int Tlen, int D) {
  using CVT = CV<T, EV>;
  const int c0 = (blockIdx.z * 256 + threadIdx.x) * EV;
  if (c0 >= D) return;
  const int t0 = blockIdx.x * SC_TT, b = blockIdx.y;
  const T *xb = x + (size_t)b * Tlen * D + c0;
  T *yb = y + (size_t)b * Tlen * D + c0;
  float wv[EV][W], bv[EV], win[W][EV];
#pragma unroll
  for (int j = 0; j < EV; ++j) {
    bv[j] = bias ? bias[c0 + j] : 0.f;
#pragma unroll
    for (int k = 0; k < W; ++k) wv[j][k] = w[(size_t)(c0 + j) * W + k];
  }
#pragma unroll
  for (int k = 0; k < W - 1; ++k) {  // win[k + 1] <- x[t0 - (W-1) + k]
    const int t = t0 - (W - 1) + k;
    CVT v;
    if (t >= 0) v = *reinterpret_cast<const CVT *>(xb + (size_t)t * D);
#pragma unroll
    for (int j = 0; j < EV; ++j) win[k + 1][j] = t >= 0 ? Num<T>::f(v.v[j]) : 0.f;
  }
  const int tend = min(t0 + SC_TT, Tlen);
  constexpr int UNF = 2 * SC_UN;
  for (int tg = t0; tg < tend; tg += UNF) {
    CVT vin[UNF];  // the group's loads are issued before any of them is used
#pragma unroll
    for (int u = 0; u < UNF; ++u)
      if (tg + u < tend) vin[u] = *reinterpret_cast<const CVT *>(xb + (size_t)(tg + u) * D);
#pragma unroll
    for (int u = 0; u < UNF; ++u) {
      const int t = tg + u;
      if (t >= tend) break;
#pragma unroll
      for (int k = 0; k < W - 1; ++k)
#pragma unroll
        for (int j = 0; j < EV; ++j) win[k][j] = win[k + 1][j];
      CVT out;
#pragma unroll
      for (int j = 0; j < EV; ++j) {
        win[W - 1][j] = Num<T>::f(vin[u].v[j]);
        float pre = bv[j];
#pragma unroll
        for (int k = 0; k < W; ++k) pre = fmaf(wv[j][k], win[k][j], pre);
        out.v[j] = Num<T>::t(ACT ? silu_f<T>(pre) : pre);
      }
      *reinterpret_cast<CVT *>(yb + (size_t)t * D) = out;
    }
  }
}

// grid (token-tile walkers, B, channel groups).  The thread recomputes pre over [t0, t0 + TT + W - 1) (the right halo
// feeds dx of its last tokens).
template <typename T, int W, bool ACT, int EV>
__global__ void __launch_bounds__(256, 3) short_conv_bwd_kernel(const T *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                                                             const T *__restrict__ dy, T *__restrict__ dx, float *__restrict__ dw,
                                                             float *__restrict__ db, int Tlen, int D) {
  using CVT = CV<T, EV>;
  const int c0 = (blockIdx.z * 256 + threadIdx.x) * EV;
  if (c0 >= D) return;
  const int b = blockIdx.y;
  const T *xb = x + (size_t)b * Tlen * D + c0, *gb = dy + (size_t)b * Tlen * D + c0;
  T *ob = dx + (size_t)b * Tlen * D + c0;
  float wv[EV][W], bv[EV], xin[W][EV], dp[W][EV], dwacc[EV][W], dbacc[EV];
#pragma unroll
  for (int j = 0; j < EV; ++j) {
    bv[j] = bias ? bias[c0 + j] : 0.f;
    dbacc[j] = 0.f;
#pragma unroll
    for (int k = 0; k < W; ++k) wv[j][k] = w[(size_t)(c0 + j) * W + k], dwacc[j][k] = 0.f;
  }
  // a block walks several token tiles (stride gridDim.x) and keeps its dweight / dbias sums in registers across them:
  // one round of atomics per thread instead of one per tile
  for (int t0 = blockIdx.x * SC_TT; t0 < Tlen; t0 += gridDim.x * SC_TT) {
#pragma unroll
  for (int j = 0; j < EV; ++j)
#pragma unroll
    for (int k = 0; k < W; ++k) dp[k][j] = 0.f;
#pragma unroll
  for (int k = 0; k < W - 1; ++k) {
    const int t = t0 - (W - 1) + k;
    CVT v;
    if (t >= 0) v = *reinterpret_cast<const CVT *>(xb + (size_t)t * D);
#pragma unroll
    for (int j = 0; j < EV; ++j) xin[k + 1][j] = t >= 0 ? Num<T>::f(v.v[j]) : 0.f;
  }
  const int tend = min(t0 + SC_TT, Tlen);
  // step s handles token t = t0 + s: computes dpre[t]; once W-1 further tokens are in, dx[t - (W-1)] is complete:
  // dx[u] = sum_w weight[w] dpre[u + (W-1) - w]  ->  with dp[k] = dpre[t - (W-1) + k]:  dx[t-(W-1)] = sum_w weight[w] dp[W-1-w]
  for (int tg = t0; tg < tend + (W - 1); tg += SC_UN) {
    CVT vin[SC_UN], gin[SC_UN];
#pragma unroll
    for (int u = 0; u < SC_UN; ++u)
      if (tg + u < Tlen && tg + u < tend + (W - 1)) {
        vin[u] = *reinterpret_cast<const CVT *>(xb + (size_t)(tg + u) * D);
        gin[u] = *reinterpret_cast<const CVT *>(gb + (size_t)(tg + u) * D);
      }
#pragma unroll
    for (int u = 0; u < SC_UN; ++u) {
      const int t = tg + u;
      if (t >= tend + (W - 1)) break;
      const bool in_seq = t < Tlen;
#pragma unroll
      for (int k = 0; k < W - 1; ++k)
#pragma unroll
        for (int j = 0; j < EV; ++j) xin[k][j] = xin[k + 1][j], dp[k][j] = dp[k + 1][j];
      const bool own = t < tend;  // tokens of the right halo belong to the next tile for dweight / dbias
#pragma unroll
      for (int j = 0; j < EV; ++j) {
        xin[W - 1][j] = in_seq ? Num<T>::f(vin[u].v[j]) : 0.f;
        float d = 0.f;
        if (in_seq) {
          float pre = bv[j];
#pragma unroll
          for (int k = 0; k < W; ++k) pre = fmaf(wv[j][k], xin[k][j], pre);
          d = Num<T>::f(gin[u].v[j]) * (ACT ? silu_grad_f<T>(pre) : 1.f);
        }
        dp[W - 1][j] = d;
        if (own) {
          dbacc[j] += d;
#pragma unroll
          for (int k = 0; k < W; ++k) dwacc[j][k] = fmaf(d, xin[k][j], dwacc[j][k]);
        }
      }
      const int uo = t - (W - 1);
      if (uo >= t0 && uo < tend) {
        CVT out;
#pragma unroll
        for (int j = 0; j < EV; ++j) {
          float a = 0.f;
#pragma unroll
          for (int k = 0; k < W; ++k) a = fmaf(wv[j][k], dp[W - 1 - k][j], a);
          out.v[j] = Num<T>::t(a);
        }
        *reinterpret_cast<CVT *>(ob + (size_t)uo * D) = out;
      }
    }
  }
  }
#pragma unroll
  for (int j = 0; j < EV; ++j) {
    if (db) atomicAdd(db + c0 + j, dbacc[j]);
#pragma unroll
    for (int k = 0; k < W; ++k) atomicAdd(dw + (size_t)(c0 + j) * W + k, dwacc[j][k]);
  }
}

// decode step: one token per sequence; cache [B, D, W] (element type T) shifted in place
template <typename T, bool ACT>
__global__ void __launch_bounds__(256) short_conv_update_kernel(const T *__restrict__ x, T *__restrict__ cache, const float *__restrict__ w,
                                                                const float *__restrict__ bias, T *__restrict__ y, int B, int D, int W) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * D) return;
  const int d = (int)(idx % D);
  T *c = cache + idx * W;
  float pre = bias ? bias[d] : 0.f;
  for (int k = 0; k < W - 1; ++k) {
    const T v = c[k + 1];
    c[k] = v;
    pre = fmaf(Num<T>::f(v), w[(size_t)d * W + k], pre);
  }
  const T xv = x[idx];
  c[W - 1] = xv;
  pre = fmaf(Num<T>::f(xv), w[(size_t)d * W + W - 1], pre);
  y[idx] = Num<T>::t(ACT ? silu_f<T>(pre) : pre);
}

template <typename T, int W>
static int launch_short_conv(bool bwd, bool act, const void *x, const float *w, const float *bias, const void *dy, void *out, float *dw, float *db,
                             int B, int Tlen, int D, cudaStream_t st) {
  const int EV = bwd ? SC_EVB : SC_EVF;
  dim3 grid(cdiv(Tlen, SC_TT), B, cdiv(D, EV * 256));
  if (bwd) {  // about two waves of blocks, each walking several token tiles
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int per_x = (int)(B * grid.z);
    const int gx = (6 * sms + per_x - 1) / per_x;  // two waves at three resident blocks per SM
    if ((int)grid.x > gx) grid.x = gx < 1 ? 1 : gx;
  }
  const T *xi = reinterpret_cast<const T *>(x), *gi = reinterpret_cast<const T *>(dy);
  T *o = reinterpret_cast<T *>(out);
  if (!bwd) {
    if (act) short_conv_fwd_kernel<T, W, true, SC_EVF><<<grid, 256, 0, st>>>(xi, w, bias, o, Tlen, D);
    else short_conv_fwd_kernel<T, W, false, SC_EVF><<<grid, 256, 0, st>>>(xi, w, bias, o, Tlen, D);
  } else {
    if (act) short_conv_bwd_kernel<T, W, true, SC_EVB><<<grid, 256, 0, st>>>(xi, w, bias, gi, o, dw, db, Tlen, D);
    else short_conv_bwd_kernel<T, W, false, SC_EVB><<<grid, 256, 0, st>>>(xi, w, bias, gi, o, dw, db, Tlen, D);
  }
  return check_launch(bwd ? "short_conv_bwd" : "short_conv_fwd");
}

template <typename T>
static int dispatch_short_conv(bool bwd, bool act, const void *x, const float *w, const float *bias, const void *dy, void *out, float *dw,
                               float *db, int B, int Tlen, int D, int W, cudaStream_t st) {
  switch (W) {
    case 2: return launch_short_conv<T, 2>(bwd, act, x, w, bias, dy, out, dw, db, B, Tlen, D, st);
    case 3: return launch_short_conv<T, 3>(bwd, act, x, w, bias, dy, out, dw, db, B, Tlen, D, st);
    case 4: return launch_short_conv<T, 4>(bwd, act, x, w, bias, dy, out, dw, db, B, Tlen, D, st);
    default: break;
  }
  set_error("short_conv: filter length %d is not supported (2, 3 or 4)", W);
  return FLAB_E_UNSUPPORTED;
}

static int short_conv_check(const void *const *ptrs, int n, int D, int dtype) {
  const int ev = 4;
  (void)dtype;
  FLAB_REQUIRE(D % ev == 0, FLAB_E_UNSUPPORTED, "short_conv: the channel count (%d) must be a multiple of %d", D, ev);
  for (int i = 0; i < n; ++i)
    FLAB_REQUIRE(!ptrs[i] || reinterpret_cast<uintptr_t>(ptrs[i]) % 16 == 0, FLAB_E_UNSUPPORTED, "short_conv: tensors must be 16-byte aligned");
  return FLAB_OK;
}

}  // namespace flab

extern "C" {

int flab_short_conv_fwd(const void *x, const float *weight, const float *bias, void *y, int B, int T, int D, int W, int silu, int dtype,
                        void *stream) {
  using namespace flab;
  if (B == 0 || T == 0) return FLAB_OK;
  FLAB_REQUIRE(x && weight && y && B > 0 && T > 0 && D > 0, FLAB_E_BADARG, "short_conv_fwd needs x, weight, y and positive B, T, D");
  const void *ptrs[2] = {x, y};
  if (int e = short_conv_check(ptrs, 2, D, dtype)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case FLAB_BF16: return dispatch_short_conv<bf16>(false, silu != 0, x, weight, bias, nullptr, y, nullptr, nullptr, B, T, D, W, st);
    case FLAB_FP16: return dispatch_short_conv<__half>(false, silu != 0, x, weight, bias, nullptr, y, nullptr, nullptr, B, T, D, W, st);
    case FLAB_FP32: return dispatch_short_conv<float>(false, silu != 0, x, weight, bias, nullptr, y, nullptr, nullptr, B, T, D, W, st);
    default: break;
  }
  set_error("short_conv_fwd: unknown dtype %d", dtype);
  return FLAB_E_BADARG;
}

int flab_short_conv_bwd(const void *x, const float *weight, const float *bias, const void *dy, void *dx, float *dweight, float *dbias, int B, int T,
                        int D, int W, int silu, int dtype, void *stream) {
  using namespace flab;
  if (B == 0 || T == 0) return FLAB_OK;
  FLAB_REQUIRE(x && weight && dy && dx && dweight && B > 0 && T > 0 && D > 0, FLAB_E_BADARG,
               "short_conv_bwd needs x, weight, dy, dx, dweight (zeroed, fp32 [D, W]) and positive B, T, D");
  FLAB_REQUIRE(!bias || dbias, FLAB_E_BADARG, "short_conv_bwd: a bias needs dbias (zeroed, fp32 [D])");
  const void *ptrs[3] = {x, dy, dx};
  if (int e = short_conv_check(ptrs, 3, D, dtype)) return e;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case FLAB_BF16: return dispatch_short_conv<bf16>(true, silu != 0, x, weight, bias, dy, dx, dweight, dbias, B, T, D, W, st);
    case FLAB_FP16: return dispatch_short_conv<__half>(true, silu != 0, x, weight, bias, dy, dx, dweight, dbias, B, T, D, W, st);
    case FLAB_FP32: return dispatch_short_conv<float>(true, silu != 0, x, weight, bias, dy, dx, dweight, dbias, B, T, D, W, st);
    default: break;
  }
  set_error("short_conv_bwd: unknown dtype %d", dtype);
  return FLAB_E_BADARG;
}

int flab_short_conv_update(const void *x, void *cache, const float *weight, const float *bias, void *y, int B, int D, int W, int silu, int dtype,
                           void *stream) {
  using namespace flab;
  if (B == 0) return FLAB_OK;
  FLAB_REQUIRE(x && cache && weight && y && B > 0 && D > 0 && W >= 1 && W <= SC_WMAX, FLAB_E_BADARG,
               "short_conv_update needs x, cache, weight, y, positive B, D and 1 <= W <= 8");
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = (long long)B * D;
  const int grid = (int)((n + 255) / 256);
#define FLAB_SC_UPD(TT)                                                                                                      \
  if (silu) short_conv_update_kernel<TT, true><<<grid, 256, 0, st>>>((const TT *)x, (TT *)cache, weight, bias, (TT *)y, B, D, W); \
  else short_conv_update_kernel<TT, false><<<grid, 256, 0, st>>>((const TT *)x, (TT *)cache, weight, bias, (TT *)y, B, D, W);      \
  return check_launch("short_conv_update");
  switch (dtype) {
    case FLAB_BF16: { FLAB_SC_UPD(bf16) }
    case FLAB_FP16: { FLAB_SC_UPD(__half) }
    case FLAB_FP32: { FLAB_SC_UPD(float) }
    default: break;
  }
#undef FLAB_SC_UPD
  set_error("short_conv_update: unknown dtype %d", dtype);
  return FLAB_E_BADARG;
}
}
