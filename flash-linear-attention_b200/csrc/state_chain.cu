// Chain of affine state transitions, S <- op(M_s) S + b_s, over the slabs of a sequence that was cut along T.
//
// Every recurrence of this path is affine in its state: a slab of tokens maps the state entering it to the state
// leaving it as S_out = M S_in + b, with M a [K, K] matrix per head that does not depend on S_in.  A scan split
// into slabs (one GPU) or ranks (sequence parallel) first obtains (M_s, b_s) of every slab, then needs the state
// entering each slab: S - 1 dependent [K,K] x [K,V] products per (sequence, head).  The products are tiny
// (4 MFLOP at K = V = 128) but serial, so they run here as ONE launch that walks all slabs, in fp32 FFMA,
// instead of a host loop of library GEMMs.  The backward chain is the transposed one, walked right to left
// (dS_in = M^T dS_out + c).  The reference has no counterpart (its unused two-level scan,
// fla/ops/common/chunk_h_split.py:164-260, covers diagonal decay only, where M is a scalar per head).
//
// grid = (ceil(V / 32), H, B); 256 threads; a CTA owns 32 state columns of one (sequence, head) for the whole
// chain: the running state [K][32] stays in shared memory, M_s is streamed through a [128][32] tile.
#include "common.cuh"

namespace flab {

constexpr int SC_VT = 32;    // state columns per CTA
constexpr int SC_RB = 128;   // rows of the product per pass (256 threads: row = tid / 2, 16 columns each)
constexpr int SC_JT = 32;    // contraction tile
constexpr int SC_PAD = SC_JT + 1;

struct ChainParams {
  const float *M, *b, *s0;
  float *s_in, *s_last;
  long long ldb;
  int B, S, H, K, V, reverse, transpose;
};

__global__ void __launch_bounds__(256) state_chain_kernel(const ChainParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int K = p.K, V = p.V;
  float *cur = reinterpret_cast<float *>(smem_raw);  // [K][SC_VT]
  float *nxt = cur + (size_t)K * SC_VT;              // [K][SC_VT]
  float *Mt = nxt + (size_t)K * SC_VT;               // [SC_RB][SC_PAD]
  const int tid = threadIdx.x;
  const int v0 = blockIdx.x * SC_VT, hd = blockIdx.y, bb = blockIdx.z;
  const int ncol = min(SC_VT, V - v0);
  // ---- the state entering the chain
  for (int e = tid; e < K * SC_VT; e += 256) {
    const int r = e / SC_VT, c = e % SC_VT;
    cur[e] = (p.s0 && c < ncol) ? p.s0[(((size_t)bb * p.H + hd) * K + r) * V + v0 + c] : 0.f;
  }
  __syncthreads();
  const int row = tid >> 1, c0 = (tid & 1) * 16;
  for (int step = 0; step < p.S; ++step) {
    const int s = p.reverse ? p.S - 1 - step : step;
    const size_t unit = ((size_t)bb * p.S + s) * p.H + hd;
    if (p.s_in) {
      float *dst = p.s_in + unit * K * V;
      for (int e = tid; e < K * SC_VT; e += 256) {
        const int r = e / SC_VT, c = e % SC_VT;
        if (c < ncol) dst[(size_t)r * V + v0 + c] = cur[e];
      }
    }
    if (step + 1 == p.S && !p.s_last) break;  // the state leaving the last slab is not wanted
    const float *M = p.M + unit * K * K;
    const float *bs = p.b + unit * K * p.ldb;
    for (int r0 = 0; r0 < K; r0 += SC_RB) {
      float acc[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) acc[c] = 0.f;
      for (int j0 = 0; j0 < K; j0 += SC_JT) {
        __syncthreads();  // the previous tile has been consumed
        // Mt[r][jj] = op(M)[r0 + r][j0 + jj]
        if (!p.transpose) {
          for (int e = tid; e < SC_RB * SC_JT; e += 256) {
            const int r = e / SC_JT, jj = e % SC_JT;
            Mt[r * SC_PAD + jj] = (r0 + r < K && j0 + jj < K) ? M[(size_t)(r0 + r) * K + j0 + jj] : 0.f;
          }
        } else {
          for (int e = tid; e < SC_RB * SC_JT; e += 256) {
            const int jj = e / SC_RB, r = e % SC_RB;  // consecutive threads walk a row of M
            Mt[r * SC_PAD + jj] = (r0 + r < K && j0 + jj < K) ? M[(size_t)(j0 + jj) * K + r0 + r] : 0.f;
          }
        }
        __syncthreads();
        const int jn = min(SC_JT, K - j0);
        for (int jj = 0; jj < jn; ++jj) {
          const float m = Mt[row * SC_PAD + jj];
          const float4 *x = reinterpret_cast<const float4 *>(cur + (size_t)(j0 + jj) * SC_VT + c0);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const float4 xv = x[q4];
            acc[4 * q4 + 0] = fmaf(m, xv.x, acc[4 * q4 + 0]);
            acc[4 * q4 + 1] = fmaf(m, xv.y, acc[4 * q4 + 1]);
            acc[4 * q4 + 2] = fmaf(m, xv.z, acc[4 * q4 + 2]);
            acc[4 * q4 + 3] = fmaf(m, xv.w, acc[4 * q4 + 3]);
          }
        }
      }
      if (r0 + row < K) {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const int col = c0 + c;
          nxt[(size_t)(r0 + row) * SC_VT + col] = col < ncol ? acc[c] + bs[(size_t)(r0 + row) * p.ldb + v0 + col] : 0.f;
        }
      }
    }
    __syncthreads();
    float *t = cur;
    cur = nxt;
    nxt = t;
  }
  if (p.s_last) {
    float *dst = p.s_last + ((size_t)bb * p.H + hd) * K * V;
    for (int e = tid; e < K * SC_VT; e += 256) {
      const int r = e / SC_VT, c = e % SC_VT;
      if (c < ncol) dst[(size_t)r * V + v0 + c] = cur[e];
    }
  }
}

}  // namespace flab

extern "C" int flab_state_chain(const float *M, const float *b, long long ldb, const float *s0, float *s_in, float *s_last, int B, int S, int H,
                                int K, int V, int flags, void *stream) {
  using namespace flab;
  FLAB_REQUIRE(M && b && (s_in || s_last), FLAB_E_BADARG, "state_chain needs M, b and at least one of s_in, s_last");
  FLAB_REQUIRE(B > 0 && S > 0 && H > 0 && K > 0 && V > 0 && ldb >= V, FLAB_E_BADARG, "state_chain: bad sizes B=%d S=%d H=%d K=%d V=%d ldb=%lld", B, S,
               H, K, V, ldb);
  FLAB_REQUIRE(K <= 256, FLAB_E_UNSUPPORTED, "state_chain: K = %d > 256", K);
  FLAB_REQUIRE(H <= 65535 && B <= 65535, FLAB_E_UNSUPPORTED, "state_chain: H and B must fit a grid dimension");
  ChainParams p{M, b, s0, s_in, s_last, ldb, B, S, H, K, V, (flags & FLAB_F_REVERSE) != 0, (flags & FLAB_F_TRANSPOSE) != 0};
  const size_t smem = (2 * (size_t)K * SC_VT + (size_t)SC_RB * SC_PAD) * sizeof(float);
  if (int e = set_smem(state_chain_kernel, smem)) return e;
  dim3 grid((V + SC_VT - 1) / SC_VT, H, B);
  state_chain_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(p);
  return check_launch("state_chain");
}
