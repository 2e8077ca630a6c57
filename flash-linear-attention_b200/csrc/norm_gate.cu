// RMS norm with a weight, times a swish gate: the step right after the chunk op in the reference's layers
// (o_norm(o, g) of GatedDeltaNet, fla/layers/gated_deltanet.py:278-280).
//   forward : rstd = 1 / sqrt(mean(x^2) + eps);  y = (x rstd w) * (g sigmoid(g))       fla/modules/fused_norm_gate.py:70-97
//   backward: yn = x rstd w;  dg = dy yn (s + g s (1 - s)), s = sigmoid(g);  dy' = dy g s;  dw += dy' xhat;
//             dx = (w dy' - xhat mean(xhat w dy')) rstd                                   fla/modules/fused_norm_gate.py:254-290
// (the reference's IS_RMS_NORM, HAS_WEIGHT branch without bias or residual).  Pure streaming, fp32 arithmetic; same
// row layout as the L2 norm: rows of 16 bytes x 2^k lanes stay in registers, several rows per warp instruction.
// dw is reduced per block (registers -> warp shuffles -> shared memory) into one partial row per block; the caller
// sums the partial rows, like the reference sums its per-program partials (fused_norm_gate.py:385-386).
#include <type_traits>

#include "common.cuh"

namespace flab {

template <typename T> struct __align__(16) V16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

// sigmoid: tanh.approx for bf16, exponential + hardware reciprocal for fp16, exponential + IEEE division for fp32
template <typename T> __device__ __forceinline__ float sigmoidf_(float x) {
  if (std::is_same<T, bf16>::value) {  // one special-function instruction; its 5e-4 absolute error is below half a bf16 ulp of the product
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
  }
  return sizeof(T) == 2 ? __fdividef(1.f, 1.f + __expf(-x)) : 1.f / (1.f + __expf(-x));
}

template <typename T, int LPR>
__global__ void __launch_bounds__(256) norm_gate_fwd_vec_kernel(const T *__restrict__ x, const T *__restrict__ g, const float *__restrict__ w,
                                                                T *__restrict__ y, float *__restrict__ rstd_out, long long rows, float eps) {
  constexpr int EV = 16 / sizeof(T), RPW = 32 / LPR, N = EV * LPR, UNROLL = 4;
  const int lane = threadIdx.x & 31, sub = lane / LPR, li = lane % LPR;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  float wv[EV];
#pragma unroll
  for (int j = 0; j < EV; ++j) wv[j] = w[li * EV + j];
  for (long long r0 = warp * RPW * UNROLL; r0 < rows; r0 += nwarps * RPW * UNROLL) {
    V16<T> xi[UNROLL], gi[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      if (r < rows) {
        xi[u] = *reinterpret_cast<const V16<T> *>(x + r * N + li * EV);
        gi[u] = *reinterpret_cast<const V16<T> *>(g + r * N + li * EV);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      float f[EV], ss = 0.f;
#pragma unroll
      for (int j = 0; j < EV; ++j) {
        f[j] = r < rows ? Num<T>::f(xi[u].v[j]) : 0.f;
        ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = 1.f / sqrtf(ss / N + eps);
      if (r < rows) {
        V16<T> out;
#pragma unroll
        for (int j = 0; j < EV; ++j) {
          const float gg = Num<T>::f(gi[u].v[j]);
          out.v[j] = Num<T>::t(f[j] * rstd * wv[j] * gg * sigmoidf_<T>(gg));
        }
        *reinterpret_cast<V16<T> *>(y + r * N + li * EV) = out;
        if (li == 0) rstd_out[r] = rstd;
      }
    }
  }
}

template <typename T, int LPR>
__global__ void __launch_bounds__(256, 2) norm_gate_bwd_vec_kernel(const T *__restrict__ x, const T *__restrict__ g, const float *__restrict__ w,
                                                                const T *__restrict__ dy, const float *__restrict__ rstd_in, T *__restrict__ dx,
                                                                T *__restrict__ dg, float *__restrict__ dw_partial, long long rows) {
  constexpr int EV = 16 / sizeof(T), RPW = 32 / LPR, N = EV * LPR;
  __shared__ float sDW[8][N];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, sub = lane / LPR, li = lane % LPR;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + wib, nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  float wv[EV], dwacc[EV];
#pragma unroll
  for (int j = 0; j < EV; ++j) wv[j] = w[li * EV + j], dwacc[j] = 0.f;
  constexpr int UNROLL = 2;  // row groups whose loads are in flight together
  for (long long r0 = warp * RPW * UNROLL; r0 < rows; r0 += nwarps * RPW * UNROLL) {
    V16<T> xv[UNROLL], gv[UNROLL], yv[UNROLL];
    float rs[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      rs[u] = 0.f;
      if (r < rows) {
        xv[u] = *reinterpret_cast<const V16<T> *>(x + r * N + li * EV);
        gv[u] = *reinterpret_cast<const V16<T> *>(g + r * N + li * EV);
        yv[u] = *reinterpret_cast<const V16<T> *>(dy + r * N + li * EV);
        rs[u] = rstd_in[r];
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      const bool on = r < rows;
      const float rstd = rs[u];
      float xhat[EV], wdy[EV], c1 = 0.f;
      V16<T> og;
#pragma unroll
      for (int j = 0; j < EV; ++j) {
        const float xf = on ? Num<T>::f(xv[u].v[j]) : 0.f, gf = on ? Num<T>::f(gv[u].v[j]) : 0.f, d = on ? Num<T>::f(yv[u].v[j]) : 0.f;
        const float s = sigmoidf_<T>(gf);
        xhat[j] = xf * rstd;
        og.v[j] = Num<T>::t(d * (xhat[j] * wv[j]) * (s + gf * s * (1.f - s)));
        const float d2 = d * gf * s;
        dwacc[j] = fmaf(d2, xhat[j], dwacc[j]);
        wdy[j] = d2 * wv[j];
        c1 = fmaf(xhat[j], wdy[j], c1);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) c1 += __shfl_xor_sync(0xffffffffu, c1, o);
      c1 *= 1.f / N;
      if (on) {
        V16<T> ox;
#pragma unroll
        for (int j = 0; j < EV; ++j) ox.v[j] = Num<T>::t((wdy[j] - xhat[j] * c1) * rstd);
        *reinterpret_cast<V16<T> *>(dx + r * N + li * EV) = ox;
        *reinterpret_cast<V16<T> *>(dg + r * N + li * EV) = og;
      }
    }
  }
  // dw: lanes with the same columns inside the warp, then the eight warps
#pragma unroll
  for (int j = 0; j < EV; ++j) {
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) dwacc[j] += __shfl_xor_sync(0xffffffffu, dwacc[j], o);
    if (sub == 0) sDW[wib][li * EV + j] = dwacc[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < N; c += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) t += sDW[wi][c];
    dw_partial[(size_t)blockIdx.x * N + c] = t;
  }
}

// any row length: one warp per row with column loops; dw through shared-memory atomics
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) norm_gate_row_kernel(const T *__restrict__ x, const T *__restrict__ g, const float *__restrict__ w,
                                                            const T *__restrict__ dy, float *__restrict__ rstd_io, T *__restrict__ out,
                                                            T *__restrict__ dg, float *__restrict__ dw_partial, long long rows, int n, float eps) {
  extern __shared__ float sdw[];
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  if (BWD) {
    for (int c = threadIdx.x; c < n; c += blockDim.x) sdw[c] = 0.f;
    __syncthreads();
  }
  for (long long r = warp; r < rows; r += nwarps) {
    const T *xr = x + r * n, *gr = g + r * n;
    if (!BWD) {
      float ss = 0.f;
      for (int c = lane; c < n; c += 32) {
        const float f = Num<T>::f(xr[c]);
        ss = fmaf(f, f, ss);
      }
      ss = warp_sum(ss);
      const float rstd = 1.f / sqrtf(ss / n + eps);
      if (lane == 0) rstd_io[r] = rstd;
      for (int c = lane; c < n; c += 32) {
        const float gg = Num<T>::f(gr[c]);
        out[r * n + c] = Num<T>::t(Num<T>::f(xr[c]) * rstd * w[c] * gg * sigmoidf_<T>(gg));
      }
    } else {
      const T *dr = dy + r * n;
      const float rstd = rstd_io[r];
      float c1 = 0.f;
      for (int c = lane; c < n; c += 32) {
        const float gf = Num<T>::f(gr[c]), s = sigmoidf_<T>(gf);
        c1 = fmaf(Num<T>::f(xr[c]) * rstd, Num<T>::f(dr[c]) * gf * s * w[c], c1);
      }
      c1 = warp_sum(c1) / n;
      for (int c = lane; c < n; c += 32) {
        const float xf = Num<T>::f(xr[c]), gf = Num<T>::f(gr[c]), d = Num<T>::f(dr[c]), s = sigmoidf_<T>(gf);
        const float xh = xf * rstd, d2 = d * gf * s, wd = d2 * w[c];
        dg[r * n + c] = Num<T>::t(d * (xh * w[c]) * (s + gf * s * (1.f - s)));
        out[r * n + c] = Num<T>::t((wd - xh * c1) * rstd);
        atomicAdd(&sdw[c], d2 * xh);
      }
    }
  }
  if (BWD) {
    __syncthreads();
    for (int c = threadIdx.x; c < n; c += blockDim.x) dw_partial[(size_t)blockIdx.x * n + c] = sdw[c];
  }
}

static int norm_gate_blocks(long long rows, int n, size_t esize, bool &vec, int &lpr) {
  const int ev = 16 / (int)esize;
  lpr = n / ev;
  vec = n % ev == 0 && lpr >= 1 && lpr <= 32 && (lpr & (lpr - 1)) == 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long passes = vec ? (rows * lpr + 31) / 32 : rows;  // warp passes
  const long long want = (passes + 15) / 16;                     // a block of 8 warps takes at least two passes per warp
  const long long cap = (long long)sms * 8;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename T>
static int launch_norm_gate(bool bwd, const void *x, const void *g, const float *w, const void *dy, float *rstd, void *out, void *dg,
                            float *dw_partial, long long rows, int n, float eps, cudaStream_t st) {
  bool vec;
  int lpr;
  const int grid = norm_gate_blocks(rows, n, sizeof(T), vec, lpr);
  const T *xi = reinterpret_cast<const T *>(x), *gi = reinterpret_cast<const T *>(g), *di = reinterpret_cast<const T *>(dy);
  T *o = reinterpret_cast<T *>(out), *dgo = reinterpret_cast<T *>(dg);
  const void *ptrs[5] = {x, g, dy, out, dg};
  for (const void *p : ptrs)
    if (p && reinterpret_cast<uintptr_t>(p) % 16 != 0) vec = false;
#define FLAB_NG_CASE(L)                                                                                         \
  case L:                                                                                                       \
    if (bwd) norm_gate_bwd_vec_kernel<T, L><<<grid, 256, 0, st>>>(xi, gi, w, di, rstd, o, dgo, dw_partial, rows); \
    else norm_gate_fwd_vec_kernel<T, L><<<grid, 256, 0, st>>>(xi, gi, w, o, rstd, rows, eps);                    \
    break;
  if (vec) {
    switch (lpr) {
      FLAB_NG_CASE(1)
      FLAB_NG_CASE(2)
      FLAB_NG_CASE(4)
      FLAB_NG_CASE(8)
      FLAB_NG_CASE(16)
      default:
        FLAB_NG_CASE(32)
    }
  } else if (bwd) {
    norm_gate_row_kernel<T, true><<<grid, 256, (size_t)n * sizeof(float), st>>>(xi, gi, w, di, rstd, o, dgo, dw_partial, rows, n, eps);
  } else {
    norm_gate_row_kernel<T, false><<<grid, 256, 0, st>>>(xi, gi, w, nullptr, rstd, o, nullptr, nullptr, rows, n, eps);
  }
#undef FLAB_NG_CASE
  return check_launch(bwd ? "rms_norm_swish_gate_bwd" : "rms_norm_swish_gate_fwd");
}

}  // namespace flab

extern "C" {

int flab_rms_norm_swish_gate_partials(long long rows, int n, int dtype) {
  bool vec;
  int lpr;
  if (rows <= 0 || n <= 0) return 1;
  return flab::norm_gate_blocks(rows, n, dtype == FLAB_FP32 ? 4 : 2, vec, lpr);
}

int flab_rms_norm_swish_gate_fwd(const void *x, const void *gate, const float *weight, void *y, float *rstd, long long rows, int n, int dtype,
                                 float eps, void *stream) {
  using namespace flab;
  if (rows == 0) return FLAB_OK;
  FLAB_REQUIRE(x && gate && weight && y && rstd && rows > 0 && n > 0, FLAB_E_BADARG, "rms_norm_swish_gate_fwd needs x, gate, weight, y, rstd");
  FLAB_REQUIRE((size_t)n * sizeof(float) <= 48 * 1024, FLAB_E_UNSUPPORTED, "rms_norm_swish_gate: rows longer than 12288 elements are not supported");
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case FLAB_BF16: return launch_norm_gate<bf16>(false, x, gate, weight, nullptr, rstd, y, nullptr, nullptr, rows, n, eps, st);
    case FLAB_FP16: return launch_norm_gate<__half>(false, x, gate, weight, nullptr, rstd, y, nullptr, nullptr, rows, n, eps, st);
    case FLAB_FP32: return launch_norm_gate<float>(false, x, gate, weight, nullptr, rstd, y, nullptr, nullptr, rows, n, eps, st);
    default: break;
  }
  set_error("rms_norm_swish_gate_fwd: unknown dtype %d", dtype);
  return FLAB_E_BADARG;
}

int flab_rms_norm_swish_gate_bwd(const void *x, const void *gate, const float *weight, const void *dy, const float *rstd, void *dx, void *dgate,
                                 float *dw_partial, long long rows, int n, int dtype, void *stream) {
  using namespace flab;
  if (rows == 0) return FLAB_OK;
  FLAB_REQUIRE(x && gate && weight && dy && rstd && dx && dgate && dw_partial && rows > 0 && n > 0, FLAB_E_BADARG,
               "rms_norm_swish_gate_bwd needs x, gate, weight, dy, rstd, dx, dgate, dw_partial");
  FLAB_REQUIRE((size_t)n * sizeof(float) <= 48 * 1024, FLAB_E_UNSUPPORTED, "rms_norm_swish_gate: rows longer than 12288 elements are not supported");
  cudaStream_t st = (cudaStream_t)stream;
  float *r = const_cast<float *>(rstd);
  switch (dtype) {
    case FLAB_BF16: return launch_norm_gate<bf16>(true, x, gate, weight, dy, r, dx, dgate, dw_partial, rows, n, 0.f, st);
    case FLAB_FP16: return launch_norm_gate<__half>(true, x, gate, weight, dy, r, dx, dgate, dw_partial, rows, n, 0.f, st);
    case FLAB_FP32: return launch_norm_gate<float>(true, x, gate, weight, dy, r, dx, dgate, dw_partial, rows, n, 0.f, st);
    default: break;
  }
  set_error("rms_norm_swish_gate_bwd: unknown dtype %d", dtype);
  return FLAB_E_BADARG;
}
}
