// Materialised attention scores of simple GLA, the optional second output of the reference's parallel form
// (parallel_simple_gla(..., output_attentions=True), fla/ops/simple_gla/parallel.py:474-544, attn written at :95-131):
//   A[b,h,i,j] = scale <q_i, k_j> exp(G_i - G_j)   for j <= i, else 0,      G = cumulative log decay of the sequence.
// A is [B,H,T,T]: quadratic in T, meant for inspection at small T, so this is a plain tiled FFMA kernel
// (fp32 accumulation, inputs of any element type); fixed-length batches only, like the reference.
// grid = (ceil(T/32), ceil(T/32), B*H), 256 threads, each thread a 2 x 2 block of a 32 x 32 tile.
#include "common.cuh"

namespace flab {

constexpr int AT = 32;  // tile edge
constexpr int AKT = 32; // contraction tile

template <typename T> __global__ void __launch_bounds__(256) simple_gla_attn_kernel(const flab_args a) {
  __shared__ float sq[AT][AKT + 1], sk[AT][AKT + 1];
  const int j0 = blockIdx.x * AT, i0 = blockIdx.y * AT;
  const int b = blockIdx.z / a.H, hd = blockIdx.z % a.H;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  T *out = reinterpret_cast<T *>(a.a) + ((size_t)b * a.H + hd) * a.T * a.T;
  if (j0 > i0 + AT - 1) {  // entirely above the diagonal
    for (int e = tid; e < AT * AT; e += 256) {
      const int i = i0 + e / AT, j = j0 + e % AT;
      if (i < a.T && j < a.T) out[(size_t)i * a.T + j] = Num<T>::t(0.f);
    }
    return;
  }
  Seq s;
  s.b = b, s.bos = 0, s.len = a.T, s.nt = 0, s.c0 = 0;
  const T *q = reinterpret_cast<const T *>(a.q) + tok_off(a, s, hd, 0, a.K);
  const T *k = reinterpret_cast<const T *>(a.k) + tok_off(a, s, hd, 0, a.K);
  const size_t ks = tok_stride(a, a.K);
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int c0 = 0; c0 < a.K; c0 += AKT) {
    for (int e = tid; e < AT * AKT; e += 256) {
      const int r = e / AKT, c = e % AKT;
      sq[r][c] = (i0 + r < a.T && c0 + c < a.K) ? Num<T>::f(q[(size_t)(i0 + r) * ks + c0 + c]) : 0.f;
      sk[r][c] = (j0 + r < a.T && c0 + c < a.K) ? Num<T>::f(k[(size_t)(j0 + r) * ks + c0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < AKT; ++c) {
      const float q0 = sq[2 * ty][c], q1 = sq[2 * ty + 1][c], k0 = sk[2 * tx][c], k1 = sk[2 * tx + 1][c];
      acc[0][0] = fmaf(q0, k0, acc[0][0]);
      acc[0][1] = fmaf(q0, k1, acc[0][1]);
      acc[1][0] = fmaf(q1, k0, acc[1][0]);
      acc[1][1] = fmaf(q1, k1, acc[1][1]);
    }
    __syncthreads();
  }
  const float *G = a.g ? reinterpret_cast<const float *>(a.g) + tok_off(a, s, hd, 0, 1) : nullptr;
  const size_t gs = tok_stride(a, 1);
#pragma unroll
  for (int di = 0; di < 2; ++di)
#pragma unroll
    for (int dj = 0; dj < 2; ++dj) {
      const int i = i0 + 2 * ty + di, j = j0 + 2 * tx + dj;
      if (i >= a.T || j >= a.T) continue;
      float x = 0.f;
      if (j <= i) x = acc[di][dj] * a.scale * (G ? expf(G[(size_t)i * gs] - G[(size_t)j * gs]) : 1.f);
      out[(size_t)i * a.T + j] = Num<T>::t(x);
    }
}

}  // namespace flab

extern "C" int flab_simple_gla_attn(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->a, FLAB_E_BADARG, "simple_gla_attn needs q, k and a");
  FLAB_REQUIRE(!a->cu_seqlens, FLAB_E_UNSUPPORTED, "simple_gla_attn: fixed-length batches only");
  FLAB_REQUIRE((long long)a->B * a->H <= 65535 && cdiv(a->T, AT) <= 65535, FLAB_E_UNSUPPORTED, "simple_gla_attn: grid too large");
  dim3 grid(cdiv(a->T, AT), cdiv(a->T, AT), a->B * a->H);
  FLAB_DISPATCH_ALL(a->dtype, T, (simple_gla_attn_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(*a)));
  return check_launch("simple_gla_attn");
}
