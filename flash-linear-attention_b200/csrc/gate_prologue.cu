// Gate / beta prologue of the gated delta rule layer (fla/layers/gated_deltanet.py:236-237):
//   beta = sigmoid(b),        g = -exp(A_log) * softplus(a + dt_bias)          (a, b: outputs of two small projections)
// in fp32, one pass over the [B,T,H] tensors, with the chunk-local cumulative sum of g (the first stage of the chunk
// op, fla/ops/gated_delta_rule/chunk.py:33) produced by the same pass.  The reference runs this as five elementwise
// PyTorch kernels plus the cumsum kernel.
//   forward : one thread per (chunk, head) walks its <= 64 tokens (the layout of the cumsum kernel)
//   backward: da = dg * (-exp(A_log)) * sigmoid(a + dt_bias),  db = dbeta * beta (1 - beta),
//             dA_log[h] = sum dg * g,  ddt_bias[h] = sum da      (per-head sums: shared-memory atomics, one global
//             atomic per head and block; the caller zeroes dA_log / ddt_bias)
#include "common.cuh"

namespace flab {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }  // torch's threshold
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(64) gdn_gate_fwd_kernel(const flab_args a, const T *__restrict__ pa, const T *__restrict__ pb,
                                                          const float *__restrict__ A_log, const float *__restrict__ dt_bias,
                                                          float *__restrict__ g, float *__restrict__ g_cum, T *__restrict__ beta) {
  const long col = (long)blockIdx.x * blockDim.x + threadIdx.x;  // (chunk, head)
  if (col >= (long)a.NT * a.H) return;
  const int c = (int)(col / a.H), h = (int)(col - (long)c * a.H);
  int n, it;
  chunk_of(a, c, n, it);
  const Seq s = seq_of(a, n);
  const int t0 = it * C, len = min(C, s.len - t0);
  const size_t base = tok_off(a, s, h, t0, 1), st = tok_stride(a, 1);
  const float neg_a = -expf(A_log[h]), bias = dt_bias ? dt_bias[h] : 0.f;
  float va[C], vb[C];
#pragma unroll
  for (int j = 0; j < C; ++j) {
    va[j] = j < len ? Num<T>::f(pa[base + (size_t)j * st]) : 0.f;
    vb[j] = j < len ? Num<T>::f(pb[base + (size_t)j * st]) : 0.f;
  }
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < C; ++j) {
    if (j < len) {
      const float gj = neg_a * softplus_f(va[j] + bias);
      acc += gj;
      g[base + (size_t)j * st] = gj;
      if (g_cum) g_cum[base + (size_t)j * st] = acc;
      beta[base + (size_t)j * st] = Num<T>::t(sigmoid_f(vb[j]));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gdn_gate_bwd_kernel(const flab_args a, const T *__restrict__ pa, const T *__restrict__ pb,
                                                           const float *__restrict__ A_log, const float *__restrict__ dt_bias,
                                                           const float *__restrict__ dg, const T *__restrict__ dbeta, T *__restrict__ da,
                                                           T *__restrict__ db, float *__restrict__ dA_log, float *__restrict__ ddt_bias) {
  extern __shared__ float sred[];  // [2][H]
  for (int e = threadIdx.x; e < 2 * a.H; e += blockDim.x) sred[e] = 0.f;
  __syncthreads();
  const long total = (long)a.B * a.T * a.H;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const int h = a.head_first ? (int)((e / a.T) % a.H) : (int)(e % a.H);
    const float na = -expf(A_log[h]), x = Num<T>::f(pa[e]) + (dt_bias ? dt_bias[h] : 0.f);
    const float dgj = dg[e];
    const float daj = dgj * na * sigmoid_f(x);
    da[e] = Num<T>::t(daj);
    const float bt = sigmoid_f(Num<T>::f(pb[e]));
    db[e] = Num<T>::t(Num<T>::f(dbeta[e]) * bt * (1.f - bt));
    atomicAdd(&sred[h], dgj * na * softplus_f(x));
    atomicAdd(&sred[a.H + h], daj);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.H; e += blockDim.x) {
    atomicAdd(&dA_log[e], sred[e]);
    if (ddt_bias) atomicAdd(&ddt_bias[e], sred[a.H + e]);
  }
}

}  // namespace flab

extern "C" {

int flab_gdn_gate_fwd(const flab_args *geo, const void *a_proj, const void *b_proj, const float *A_log, const float *dt_bias, float *g,
                      float *g_cumsum, void *beta, void *stream) {
  using namespace flab;
  if (int e = check_common(geo)) return e;
  FLAB_REQUIRE(a_proj && b_proj && A_log && g && beta, FLAB_E_BADARG, "gdn_gate_fwd needs a_proj, b_proj, A_log, g and beta");
  FLAB_REQUIRE(geo->NT > 0, FLAB_E_BADARG, "gdn_gate_fwd: NT must be positive");
  const long cols = (long)geo->NT * geo->H;
  const unsigned blocks = (unsigned)((cols + 63) / 64);
  FLAB_DISPATCH_ALL(geo->dtype, T,
                    (gdn_gate_fwd_kernel<T><<<blocks, 64, 0, (cudaStream_t)stream>>>(*geo, (const T *)a_proj, (const T *)b_proj, A_log, dt_bias, g,
                                                                                    g_cumsum, (T *)beta)));
  return check_launch("gdn_gate_fwd");
}

int flab_gdn_gate_bwd(const flab_args *geo, const void *a_proj, const void *b_proj, const float *A_log, const float *dt_bias, const float *dg,
                      const void *dbeta, void *da, void *db, float *dA_log, float *ddt_bias, void *stream) {
  using namespace flab;
  if (int e = check_common(geo)) return e;
  FLAB_REQUIRE(a_proj && b_proj && A_log && dg && dbeta && da && db && dA_log, FLAB_E_BADARG,
               "gdn_gate_bwd needs a_proj, b_proj, A_log, dg, dbeta, da, db and dA_log");
  FLAB_REQUIRE(geo->H <= 4096, FLAB_E_UNSUPPORTED, "gdn_gate_bwd: H = %d > 4096", geo->H);
  const long total = (long)geo->B * geo->T * geo->H;
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  const size_t smem = 2 * (size_t)geo->H * sizeof(float);
  FLAB_DISPATCH_ALL(geo->dtype, T,
                    (gdn_gate_bwd_kernel<T><<<(unsigned)blocks, 256, smem, (cudaStream_t)stream>>>(
                        *geo, (const T *)a_proj, (const T *)b_proj, A_log, dt_bias, dg, (const T *)dbeta, (T *)da, (T *)db, dA_log, ddt_bias)));
  return check_launch("gdn_gate_bwd");
}
}
