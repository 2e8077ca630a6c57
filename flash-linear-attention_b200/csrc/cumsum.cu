// Gate cumulative sums: chunk-local (64-token chunks, restarted at every sequence start) and
// whole-sequence, forward or reverse, scalar [B,T,H] or vector [B,T,H,S] inputs.
// Pure HBM streaming work: one thread owns one (chunk|sequence, head[, channel]) column and walks
// it serially; adjacent threads touch adjacent addresses (heads or channels), so every warp
// access is a contiguous segment in the seq-first layout.
#include "common.cuh"

namespace flab {

// x: element type T, y: fp32. `inner` = H (scalar) or H*S (vector) columns per token in seq-first
// layout; in head-first layout a column (b,h[,s]) is strided by `S` (1 for scalar) along tokens.
template <typename T, bool LOCAL>
__global__ void cumsum_kernel(const flab_args a, const T *__restrict__ x, float *__restrict__ y, int S) {
  const int HS = a.H * S;
  const long col = (long)blockIdx.x * blockDim.x + threadIdx.x;  // (unit, h, s)
  const long units = LOCAL ? (long)a.NT : (long)a.N;
  if (col >= units * HS) return;
  const int unit = (int)(col / HS);
  const int hs = (int)(col - (long)unit * HS);
  const int h = hs / S, sc = hs - h * S;
  int n, t0, t1;
  Seq s;
  if (LOCAL) {
    int it;
    chunk_of(a, unit, n, it);
    s = seq_of(a, n);
    t0 = it * C;
    t1 = min(t0 + C, s.len);
  } else {
    s = seq_of(a, unit);
    t0 = 0;
    t1 = s.len;
  }
  const size_t base = tok_off(a, s, h, 0, S) + sc;
  const size_t st = tok_stride(a, S);
  float acc = 0.f;
  if (LOCAL) {
    // a chunk is at most 64 tokens: fetch the whole column first (independent loads, all in flight together),
    // then run the dependent chain over registers
    const bool rev = (a.flags & FLAB_F_REVERSE) != 0;
    const int len = t1 - t0;
    float v[C];
#pragma unroll
    for (int j = 0; j < C; ++j) v[j] = j < len ? Num<T>::f(x[base + (size_t)(rev ? t1 - 1 - j : t0 + j) * st]) : 0.f;
#pragma unroll
    for (int j = 0; j < C; ++j) {
      acc += v[j];
      if (j < len) y[base + (size_t)(rev ? t1 - 1 - j : t0 + j) * st] = acc;
    }
    return;
  }
  if (a.flags & FLAB_F_REVERSE) {
    for (int t = t1 - 1; t >= t0; --t) {
      acc += Num<T>::f(x[base + (size_t)t * st]);
      y[base + (size_t)t * st] = acc;
    }
  } else {
    for (int t = t0; t < t1; ++t) {
      acc += Num<T>::f(x[base + (size_t)t * st]);
      y[base + (size_t)t * st] = acc;
    }
  }
}

template <bool LOCAL> static int launch_cumsum(const flab_args *a, int S, void *stream) {
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->x && a->y, FLAB_E_BADARG, "cumsum needs x and y");
  FLAB_REQUIRE(S > 0, FLAB_E_BADARG, "cumsum: S must be positive");
  if (LOCAL) FLAB_REQUIRE(a->NT > 0, FLAB_E_BADARG, "cumsum: NT must be positive");
  long cols = (long)(LOCAL ? a->NT : a->N) * a->H * S;
  const int threads = LOCAL ? 64 : 128;
  long blocks = (cols + threads - 1) / threads;
  FLAB_DISPATCH_ALL(a->dtype, T,
                    cumsum_kernel<T, LOCAL><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
                        *a, (const T *)a->x, (float *)a->y, S));
  return check_launch("cumsum");
}

}  // namespace flab

extern "C" {
int flab_chunk_local_cumsum_scalar(const flab_args *a, void *stream) { return flab::launch_cumsum<true>(a, 1, stream); }
int flab_chunk_local_cumsum_vector(const flab_args *a, void *stream) {
  return flab::launch_cumsum<true>(a, a ? a->S : 0, stream);
}
int flab_chunk_global_cumsum_scalar(const flab_args *a, void *stream) { return flab::launch_cumsum<false>(a, 1, stream); }
int flab_chunk_global_cumsum_vector(const flab_args *a, void *stream) {
  return flab::launch_cumsum<false>(a, a ? a->S : 0, stream);
}
}
