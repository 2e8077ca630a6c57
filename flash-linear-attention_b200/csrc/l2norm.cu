// Row-wise L2 normalisation, the step right before the chunk ops in the reference's layers (q and k of
// GatedDeltaNet / DeltaNet): y = x / sqrt(sum(x^2) + eps) over the last dimension.
//   forward : fla/modules/l2norm.py:15-36   (l2norm_fwd_kernel)
//   backward: fla/modules/l2norm.py:50-85   dx = dy * r - sum(dy * x) * r / (var + eps) * x,  r = 1 / sqrt(var + eps)
// Pure HBM streaming: a row of N elements is read once (forward) or two rows once (backward) and one row written.
// Rows whose length is 16 bytes x a power of two <= 32 lanes are held in registers, one 16-byte vector per lane and
// several rows per warp instruction, four row groups in flight per warp; other lengths take one warp per row with a
// column loop.  Arithmetic in fp32, inputs and outputs bf16 / fp16 / fp32 (the output type may differ).
#include "common.cuh"

namespace flab {

template <typename T> struct __align__(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename TI, typename TO, int LPR /* lanes per row */>
__global__ void __launch_bounds__(256) l2norm_fwd_vec_kernel(const TI *__restrict__ x, TO *__restrict__ y, long long rows, float eps) {
  constexpr int EV = 16 / sizeof(TI), RPW = 32 / LPR, N = EV * LPR, UNROLL = 4;
  const int lane = threadIdx.x & 31, sub = lane / LPR, li = lane % LPR;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r0 = warp * RPW * UNROLL; r0 < rows; r0 += nwarps * RPW * UNROLL) {
    Vec16<TI> in[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      if (r < rows) in[u] = *reinterpret_cast<const Vec16<TI> *>(x + r * N + li * EV);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      float f[EV], ss = 0.f;
#pragma unroll
      for (int j = 0; j < EV; ++j) {
        f[j] = r < rows ? Num<TI>::f(in[u].v[j]) : 0.f;
        ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = 1.f / sqrtf(ss + eps);
      if (r < rows) {
        TO *dst = y + r * N + li * EV;
#pragma unroll
        for (int h = 0; h < (int)(EV * sizeof(TO) / 16); ++h) {
          Vec16<TO> out;
#pragma unroll
          for (int j = 0; j < Vec16<TO>::N; ++j) out.v[j] = Num<TO>::t(f[h * Vec16<TO>::N + j] * rstd);
          *reinterpret_cast<Vec16<TO> *>(dst + h * Vec16<TO>::N) = out;
        }
        if (EV * sizeof(TO) < 16) {  // narrower output than input (fp32 -> 16-bit): four 2-byte stores
#pragma unroll
          for (int j = 0; j < EV; ++j) dst[j] = Num<TO>::t(f[j] * rstd);
        }
      }
    }
  }
}

template <typename T, int LPR>
__global__ void __launch_bounds__(256) l2norm_bwd_vec_kernel(const T *__restrict__ x, const T *__restrict__ dy, T *__restrict__ dx, long long rows,
                                                             float eps) {
  constexpr int EV = 16 / sizeof(T), RPW = 32 / LPR, N = EV * LPR, UNROLL = 2;
  const int lane = threadIdx.x & 31, sub = lane / LPR, li = lane % LPR;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r0 = warp * RPW * UNROLL; r0 < rows; r0 += nwarps * RPW * UNROLL) {
    Vec16<T> xi[UNROLL], gi[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      if (r < rows) {
        xi[u] = *reinterpret_cast<const Vec16<T> *>(x + r * N + li * EV);
        gi[u] = *reinterpret_cast<const Vec16<T> *>(dy + r * N + li * EV);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long r = r0 + u * RPW + sub;
      float f[EV], g[EV], ss = 0.f, dot = 0.f;
#pragma unroll
      for (int j = 0; j < EV; ++j) {
        f[j] = r < rows ? Num<T>::f(xi[u].v[j]) : 0.f;
        g[j] = r < rows ? Num<T>::f(gi[u].v[j]) : 0.f;
        ss = fmaf(f[j], f[j], ss);
        dot = fmaf(f[j], g[j], dot);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
      }
      const float rstd = 1.f / sqrtf(ss + eps), c = dot * (1.f / (ss + eps)) * rstd;
      if (r < rows) {
        Vec16<T> out;
#pragma unroll
        for (int j = 0; j < EV; ++j) out.v[j] = Num<T>::t(g[j] * rstd - c * f[j]);
        *reinterpret_cast<Vec16<T> *>(dx + r * N + li * EV) = out;
      }
    }
  }
}

// any row length: one warp per row, two passes over the row (the second one hits L1 / L2)
template <typename TI, typename TO, bool BWD>
__global__ void __launch_bounds__(256) l2norm_row_kernel(const TI *__restrict__ x, const TI *__restrict__ dy, TO *__restrict__ out, long long rows,
                                                         int n, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = warp; r < rows; r += nwarps) {
    const TI *xr = x + r * n, *gr = BWD ? dy + r * n : nullptr;
    float ss = 0.f, dot = 0.f;
    for (int c = lane; c < n; c += 32) {
      const float f = Num<TI>::f(xr[c]);
      ss = fmaf(f, f, ss);
      if (BWD) dot = fmaf(f, Num<TI>::f(gr[c]), dot);
    }
    ss = warp_sum(ss);
    if (BWD) dot = warp_sum(dot);
    const float rstd = 1.f / sqrtf(ss + eps), cc = dot * (1.f / (ss + eps)) * rstd;
    for (int c = lane; c < n; c += 32) {
      const float f = Num<TI>::f(xr[c]);
      out[r * n + c] = Num<TO>::t(BWD ? Num<TI>::f(gr[c]) * rstd - cc * f : f * rstd);
    }
  }
}

static int l2norm_grid(long long work_items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (work_items + 7) / 8;  // 8 warps per block
  const long long cap = (long long)sms * 8;     // eight resident blocks of 256 threads per SM
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename TI, typename TO> static int launch_l2norm_fwd(const void *x, void *y, long long rows, int n, float eps, cudaStream_t st) {
  constexpr int EV = 16 / sizeof(TI);
  const bool aligned = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
  const int lpr = n / EV;
  const TI *xi = reinterpret_cast<const TI *>(x);
  TO *yo = reinterpret_cast<TO *>(y);
  if (aligned && n % EV == 0 && lpr >= 1 && lpr <= 32 && (lpr & (lpr - 1)) == 0 && sizeof(TO) <= sizeof(TI) * 2) {
    const int grid = l2norm_grid((rows * lpr + 31) / 32 / 4 + 1);
    switch (lpr) {
      case 1: l2norm_fwd_vec_kernel<TI, TO, 1><<<grid, 256, 0, st>>>(xi, yo, rows, eps); break;
      case 2: l2norm_fwd_vec_kernel<TI, TO, 2><<<grid, 256, 0, st>>>(xi, yo, rows, eps); break;
      case 4: l2norm_fwd_vec_kernel<TI, TO, 4><<<grid, 256, 0, st>>>(xi, yo, rows, eps); break;
      case 8: l2norm_fwd_vec_kernel<TI, TO, 8><<<grid, 256, 0, st>>>(xi, yo, rows, eps); break;
      case 16: l2norm_fwd_vec_kernel<TI, TO, 16><<<grid, 256, 0, st>>>(xi, yo, rows, eps); break;
      default: l2norm_fwd_vec_kernel<TI, TO, 32><<<grid, 256, 0, st>>>(xi, yo, rows, eps); break;
    }
  } else {
    l2norm_row_kernel<TI, TO, false><<<l2norm_grid(rows), 256, 0, st>>>(xi, nullptr, yo, rows, n, eps);
  }
  return check_launch("l2norm_fwd");
}

template <typename T> static int launch_l2norm_bwd(const void *x, const void *dy, void *dx, long long rows, int n, float eps, cudaStream_t st) {
  constexpr int EV = 16 / sizeof(T);
  const bool aligned = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(dy) % 16 == 0 && reinterpret_cast<uintptr_t>(dx) % 16 == 0;
  const int lpr = n / EV;
  const T *xi = reinterpret_cast<const T *>(x), *gi = reinterpret_cast<const T *>(dy);
  T *o = reinterpret_cast<T *>(dx);
  if (aligned && n % EV == 0 && lpr >= 1 && lpr <= 32 && (lpr & (lpr - 1)) == 0) {
    const int grid = l2norm_grid((rows * lpr + 31) / 32 / 2 + 1);
    switch (lpr) {
      case 1: l2norm_bwd_vec_kernel<T, 1><<<grid, 256, 0, st>>>(xi, gi, o, rows, eps); break;
      case 2: l2norm_bwd_vec_kernel<T, 2><<<grid, 256, 0, st>>>(xi, gi, o, rows, eps); break;
      case 4: l2norm_bwd_vec_kernel<T, 4><<<grid, 256, 0, st>>>(xi, gi, o, rows, eps); break;
      case 8: l2norm_bwd_vec_kernel<T, 8><<<grid, 256, 0, st>>>(xi, gi, o, rows, eps); break;
      case 16: l2norm_bwd_vec_kernel<T, 16><<<grid, 256, 0, st>>>(xi, gi, o, rows, eps); break;
      default: l2norm_bwd_vec_kernel<T, 32><<<grid, 256, 0, st>>>(xi, gi, o, rows, eps); break;
    }
  } else {
    l2norm_row_kernel<T, T, true><<<l2norm_grid(rows), 256, 0, st>>>(xi, gi, o, rows, n, eps);
  }
  return check_launch("l2norm_bwd");
}

}  // namespace flab

extern "C" {

int flab_l2norm_fwd(const void *x, void *y, long long rows, int n, int in_dtype, int out_dtype, float eps, void *stream) {
  using namespace flab;
  if (rows == 0) return FLAB_OK;
  FLAB_REQUIRE(x && y && rows > 0 && n > 0, FLAB_E_BADARG, "l2norm_fwd needs x, y, rows >= 0 and n > 0");
  cudaStream_t st = (cudaStream_t)stream;
  const int key = in_dtype * 3 + out_dtype;
  switch (key) {
    case FLAB_BF16 * 3 + FLAB_BF16: return launch_l2norm_fwd<bf16, bf16>(x, y, rows, n, eps, st);
    case FLAB_BF16 * 3 + FLAB_FP32: return launch_l2norm_fwd<bf16, float>(x, y, rows, n, eps, st);
    case FLAB_FP16 * 3 + FLAB_FP16: return launch_l2norm_fwd<__half, __half>(x, y, rows, n, eps, st);
    case FLAB_FP16 * 3 + FLAB_FP32: return launch_l2norm_fwd<__half, float>(x, y, rows, n, eps, st);
    case FLAB_FP32 * 3 + FLAB_FP32: return launch_l2norm_fwd<float, float>(x, y, rows, n, eps, st);
    case FLAB_FP32 * 3 + FLAB_BF16: return launch_l2norm_fwd<float, bf16>(x, y, rows, n, eps, st);
    case FLAB_FP32 * 3 + FLAB_FP16: return launch_l2norm_fwd<float, __half>(x, y, rows, n, eps, st);
    default: break;
  }
  set_error("l2norm_fwd: element types %d -> %d are not supported", in_dtype, out_dtype);
  return FLAB_E_UNSUPPORTED;
}

int flab_l2norm_bwd(const void *x, const void *dy, void *dx, long long rows, int n, int dtype, float eps, void *stream) {
  using namespace flab;
  if (rows == 0) return FLAB_OK;
  FLAB_REQUIRE(x && dy && dx && rows > 0 && n > 0, FLAB_E_BADARG, "l2norm_bwd needs x, dy, dx, rows >= 0 and n > 0");
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case FLAB_BF16: return launch_l2norm_bwd<bf16>(x, dy, dx, rows, n, eps, st);
    case FLAB_FP16: return launch_l2norm_bwd<__half>(x, dy, dx, rows, n, eps, st);
    case FLAB_FP32: return launch_l2norm_bwd<float>(x, dy, dx, rows, n, eps, st);
    default: break;
  }
  set_error("l2norm_bwd: unknown dtype %d", dtype);
  return FLAB_E_BADARG;
}
}
