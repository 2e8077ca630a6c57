// Token-recurrent kernels (decode and the reference's test oracles).
//
// Forward: the [K x V] state is register resident, rows split over the warps and 4 columns per lane
// (512-byte row segments per warp access).  The state is read once and written once per call -
// decode (T = 1) is a pure stream over the state and runs at HBM speed.
//   generic gates g / gk / gv:  fla/ops/common/fused_recurrent.py:27-128
//   delta rule (optional scalar gate): fla/ops/delta_rule/fused_recurrent.py:19-109,
//                                      fla/ops/gated_delta_rule/fused_recurrent.py:19-110
// Backward (training-time check path): the state lives in shared memory and every token does row
// and column reductions over it (fla/ops/common/fused_recurrent.py:145-319,
// fla/ops/delta_rule/fused_recurrent.py:118-290).
#include "tc.cuh"

FLAB_TC_DEFINE_ERROR_WORD(recurrent_error)

namespace flab {

constexpr int RC_V = 128;     // value columns per CTA
constexpr int RC_WARPS = 16;  // the K rows of the state are split over the warps

// ------------------------------------------------------------------------------------------------
// forward.  CTA = (sequence, head, 128-wide V tile), 16 warps.  Warp w owns RPW consecutive state rows,
// lane l owns 4 consecutive columns, so a warp instruction moves one full 512-byte row segment and a warp
// streams RPW * 512 contiguous bytes of the fp32 state: decode (T = 1) is one coalesced pass over it.
// The reductions over K (o = S^T q and the delta-rule correction S^T k) are thread-local over the
// warp's rows, then summed across the warps through shared memory (one barrier pair per token).
// The delta rule needs both reductions before the rank-1 update; using
//   o = (S + k v'^T)^T q = S^T q + v' (k.q)
// both are taken in the same pass over the (decayed) state.
// ------------------------------------------------------------------------------------------------
template <typename T, int RPW, bool DELTA>
__global__ void __launch_bounds__(RC_WARPS * 32, (RPW <= 8 ? 2 : 1)) recurrent_fwd_kernel(const flab_args a) {
  __shared__ float sQ[256], sK[256], sE[256];  // q*scale, k, exp(gk) of the current token
  __shared__ float sRed[2][RC_WARPS][RC_V];    // cross-warp partial sums
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.y / a.H, hd = blockIdx.y % a.H;
  const Seq s = seq_of(a, n);
  const int K = a.K, V = a.V;
  const int c0 = blockIdx.x * RC_V + 4 * lane;  // first of this lane's 4 columns
  const int r0 = warp * RPW;
  const bool rev = (a.flags & FLAB_F_REVERSE) != 0;
  const bool beta_vec = (a.flags & FLAB_F_BETA_VECTOR) != 0;
  const bool vec4 = (V % 4 == 0);  // rows of h0 / ht are then 16-byte aligned at every c0

  float S[RPW][4];
  const size_t st_off = ((size_t)n * a.H + hd) * K * V;
  const float *h0 = reinterpret_cast<const float *>(a.h0);
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int kk = r0 + i;
    S[i][0] = S[i][1] = S[i][2] = S[i][3] = 0.f;
    if (h0 && kk < K) {
      const float *p = h0 + st_off + (size_t)kk * V + c0;
      if (vec4 && c0 + 3 < V) {
        const float4 x = *reinterpret_cast<const float4 *>(p);
        S[i][0] = x.x, S[i][1] = x.y, S[i][2] = x.z, S[i][3] = x.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c0 + j < V) S[i][j] = p[j];
      }
    }
  }
  const T *q = reinterpret_cast<const T *>(a.q), *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v);
  const float *g = reinterpret_cast<const float *>(a.g), *gk = reinterpret_cast<const float *>(a.gk),
              *gv = reinterpret_cast<const float *>(a.gv);
  const T *beta = reinterpret_cast<const T *>(a.beta);

  for (int i_t = 0; i_t < s.len; ++i_t) {
    const int t = rev ? s.len - 1 - i_t : i_t;
    const size_t ok_ = tok_off(a, s, hd, t, K), ov = tok_off(a, s, hd, t, V), o1 = tok_off(a, s, hd, t, 1);
    __syncthreads();  // previous token's shared vectors and partial sums are consumed
    for (int i = tid; i < K; i += RC_WARPS * 32) {
      sQ[i] = Num<T>::f(q[ok_ + i]) * a.scale;
      sK[i] = Num<T>::f(k[ok_ + i]);
      if (gk) sE[i] = expf(gk[ok_ + i]);
    }
    float vv[4], dec[4], bb[4];
    const float eg = g ? expf(g[o1]) : 1.f;
    const float bs = (DELTA && beta && !beta_vec) ? Num<T>::f(beta[o1]) : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool ok = c0 + j < V;
      vv[j] = ok ? Num<T>::f(v[ov + c0 + j]) : 0.f;
      dec[j] = (gv && ok) ? eg * expf(gv[ov + c0 + j]) : eg;
      bb[j] = (DELTA && beta && beta_vec) ? (ok ? Num<T>::f(beta[ov + c0 + j]) : 0.f) : bs;
    }
    __syncthreads();
    float pq[4] = {0.f, 0.f, 0.f, 0.f}, pk[4] = {0.f, 0.f, 0.f, 0.f};
    if (!DELTA) {
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const int kk = r0 + i;
        if (kk < K) {
          const float e = gk ? sE[kk] : 1.f, kv = sK[kk], qv = sQ[kk];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            S[i][j] = S[i][j] * (e * dec[j]) + kv * vv[j];
            pq[j] = fmaf(S[i][j], qv, pq[j]);
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const int kk = r0 + i;
        if (kk < K) {
          const float kv = sK[kk], qv = sQ[kk];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            S[i][j] *= dec[j];
            pk[j] = fmaf(S[i][j], kv, pk[j]);
            pq[j] = fmaf(S[i][j], qv, pq[j]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sRed[0][warp][4 * lane + j] = pq[j];
      if (DELTA) sRed[1][warp][4 * lane + j] = pk[j];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float x = 0.f, y = 0.f;
#pragma unroll
      for (int w = 0; w < RC_WARPS; ++w) {
        x += sRed[0][w][4 * lane + j];
        if (DELTA) y += sRed[1][w][4 * lane + j];
      }
      pq[j] = x;
      pk[j] = y;
    }
    if (DELTA) {
      // k . q over all K (every warp computes it; q is already scaled)
      float kq = 0.f;
      for (int i = lane; i < K; i += 32) kq = fmaf(sK[i], sQ[i], kq);
      kq = warp_sum(kq);
      float vn[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float u_ = vv[j] - pk[j];
        if (a.u && warp == 0 && c0 + j < V) reinterpret_cast<T *>(a.u)[ov + c0 + j] = Num<T>::t(u_);
        vn[j] = u_ * bb[j];
        pq[j] = fmaf(vn[j], kq, pq[j]);
      }
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const int kk = r0 + i;
        if (kk < K) {
          const float kv = sK[kk];
#pragma unroll
          for (int j = 0; j < 4; ++j) S[i][j] = fmaf(kv, vn[j], S[i][j]);
        }
      }
    }
    if (warp == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + j < V) {
          if (DELTA) reinterpret_cast<T *>(a.o)[ov + c0 + j] = Num<T>::t(pq[j]);
          else reinterpret_cast<float *>(a.o)[ov + c0 + j] = pq[j];
        }
    }
  }
  float *ht = reinterpret_cast<float *>(a.ht);
  if (ht) {
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const int kk = r0 + i;
      if (kk < K) {
        float *p = ht + st_off + (size_t)kk * V + c0;
        if (vec4 && c0 + 3 < V) {
          *reinterpret_cast<float4 *>(p) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c0 + j < V) p[j] = S[i][j];
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Streaming variant of the delta-rule recurrence for V == 128, K <= 128 with an initial state (the
// decode configuration).  Persistent CTAs, one per SM, two groups of 8 consumer warps (each group works on
// alternate items, so that four warps per scheduler hide each other's latencies); no producer warp:
//  * the 64 KB fp32 state tile of each (sequence, head) arrives through a 3-deep ring of bulk async
//    copies, one 8 KB piece (16 rows) per consumer warp with its own mbarrier: a warp waits for its piece only,
//    drains it into registers and at once asks for the same piece of the tile three items ahead, so the
//    copies in flight never wait for a barrier among warps; the loads carry an evict-first L2 hint and the
//    state is stored with streaming stores (neither is read again by this kernel);
//  * a consumer warp owns 16 state rows, a lane 4 columns; the k / q values of the warp's rows sit in
//    one register per lane (lanes 0-15: k, lanes 16-31: q*scale) and are broadcast with shuffles; they
//    and v, g, beta are fetched one token ahead, so no global-load latency is exposed;
//  * one named barrier per token (the cross-warp reduction of S^T k, S^T q and k.q, double buffered);
//  * the new state goes straight from registers to global memory with 512-byte warp stores.
// ------------------------------------------------------------------------------------------------
constexpr int RS_STAGES = 3;

__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar))
               : "memory");
}
// the same copy with an L2 eviction policy (made by createpolicy) for data that is read exactly once
__device__ __forceinline__ void bulk_load_hint(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                   tc::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(bar)), "l"(policy)
               : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void st_streaming(float *dst, float4 x) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
}

// VARIANT bits (the launcher picks): 1 = per-warp pieces of the ring, 2 = evict-first loads, 4 = streaming stores of
// the new state.  With FLAB_F_DESCENDING the tiles are walked from the last to the first: the state a decode step
// reads is the one the previous step wrote, and the tiles written last are still in L2 when the next step starts.
template <typename T, int VARIANT>
__global__ void __launch_bounds__(512, 1) recurrent_stream_kernel(const flab_args a, int n_items) {
  using namespace tc;
  constexpr int RPW = 16;
  constexpr bool PIECES = (VARIANT & 1) != 0, HINT = (VARIANT & 2) != 0, STREAM_ST = (VARIANT & 4) != 0;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  float *sState = reinterpret_cast<float *>(smem_raw);  // [RS_STAGES][128][128]
  __shared__ __align__(16) float sRedAll[2][2][2][8][RC_V];  // [group][parity][S^T q | S^T k][warp][column]
  __shared__ float sKQAll[2][2][8];
  __shared__ volatile int fail_snap[2][2];
  __shared__ uint64_t full[RS_STAGES][8];  // [slot][piece]; the whole-tile form uses piece 0 only
  __shared__ volatile int fail_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = a.K, V = a.V;  // V == 128
  const uint32_t tile_bytes = (uint32_t)K * RC_V * sizeof(float);
  const float *h0 = reinterpret_cast<const float *>(a.h0);
  float *ht = reinterpret_cast<float *>(a.ht);
  const T *q = reinterpret_cast<const T *>(a.q), *k = reinterpret_cast<const T *>(a.k), *v = reinterpret_cast<const T *>(a.v);
  const float *g = reinterpret_cast<const float *>(a.g);
  const T *beta = reinterpret_cast<const T *>(a.beta);
  const bool beta_vec = (a.flags & FLAB_F_BETA_VECTOR) != 0;
  const int n_local = n_items > (int)blockIdx.x ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const bool descending = (a.flags & FLAB_F_DESCENDING) != 0;
  auto item_of = [&](int li) -> int {  // global (sequence, head) index of this CTA's li-th item
    const int up = (int)blockIdx.x + li * (int)gridDim.x;
    return descending ? n_items - 1 - up : up;
  };
  const uint64_t pol = HINT ? policy_evict_first() : 0;
  auto copy_in = [&](void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    mbar_expect_tx(bar, bytes);
    if (HINT) bulk_load_hint(dst, src, bytes, bar, pol);
    else bulk_load(dst, src, bytes, bar);
  };
  auto refill = [&](int i) {  // one thread: tile of local item i -> its slot
    if (i >= n_local) return;
    const int st = i % RS_STAGES;
    copy_in(sState + (size_t)st * 128 * RC_V, h0 + (size_t)item_of(i) * K * V, tile_bytes, &full[st][0]);
  };
  auto refill_piece = [&](int i, int w) {  // one thread: rows 16 w .. 16 w + 15 of the tile of local item i
    const int rows = min(RPW, K - w * RPW);
    if (i >= n_local || rows <= 0) return;
    const int st = i % RS_STAGES;
    copy_in(sState + (size_t)st * 128 * RC_V + (size_t)w * RPW * RC_V,
            h0 + (size_t)item_of(i) * K * V + (size_t)w * RPW * RC_V, (uint32_t)rows * RC_V * sizeof(float), &full[st][w]);
  };
  if (tid == 0) {
    for (int i = 0; i < RS_STAGES; ++i)
      for (int w = 0; w < 8; ++w) mbar_init(&full[i][w], 1);
    fail_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    for (int i = 0; i < RS_STAGES; ++i) {
      if (PIECES) {
        for (int w = 0; w < 8; ++w) refill_piece(i, w);
      } else {
        refill(i);
      }
    }
  }
  __syncthreads();
  // ---------------------------------------------------------------------------------- consumers
  const int grp = warp >> 3, gw = warp & 7;
  float (*sRed)[2][8][RC_V] = sRedAll[grp];
  float (*sKQ)[8] = sKQAll[grp];
  const int c0 = 4 * lane, r0 = gw * RPW;
  float n_kq = 0.f, n_v[4] = {0.f, 0.f, 0.f, 0.f}, n_b[4] = {1.f, 1.f, 1.f, 1.f}, n_eg = 1.f;
  auto fetch = [&](int li, int i_t) {  // vectors of token i_t of local item li -> registers
    if (li >= n_local) return;
    const int item = item_of(li);
    const int n = item / a.H, hd = item % a.H;
    const Seq s = seq_of(a, n);
    if (i_t >= s.len) return;
    const size_t ok_ = tok_off(a, s, hd, i_t, K), ov = tok_off(a, s, hd, i_t, V), o1 = tok_off(a, s, hd, i_t, 1);
    const int row = r0 + (lane & 15);
    n_kq = 0.f;
    if (row < K) n_kq = lane < 16 ? Num<T>::f(k[ok_ + row]) : Num<T>::f(q[ok_ + row]) * a.scale;
    n_eg = g ? expf(g[o1]) : 1.f;
    const float bs = (beta && !beta_vec) ? Num<T>::f(beta[o1]) : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      n_v[j] = Num<T>::f(v[ov + c0 + j]);
      n_b[j] = (beta && beta_vec) ? Num<T>::f(beta[ov + c0 + j]) : bs;
    }
  };
  fetch(grp, 0);
  int par = 0;
  for (int i = grp; i < n_local; i += 2) {
    const int item = item_of(i);
    const int n = item / a.H, hd = item % a.H;
    const Seq s = seq_of(a, n);
    const int st = i % RS_STAGES;
    if ((!PIECES || r0 < K) && !mbar_wait(&full[st][PIECES ? gw : 0], (i / RS_STAGES) & 1)) {
      atomicCAS(&tu_tc_error, 0, 20);
      fail_flag = 1;
    }

    float S[RPW][4];
    const float *tile = sState + (size_t)st * 128 * RC_V;
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int kk = r0 + r;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kk < K) x = *reinterpret_cast<const float4 *>(tile + (size_t)kk * RC_V + c0);
      S[r][0] = x.x, S[r][1] = x.y, S[r][2] = x.z, S[r][3] = x.w;
    }
    if (PIECES) {  // this warp's piece is in registers: ask for the same piece three items ahead, before any barrier
      __syncwarp();
      if (lane == 0) refill_piece(i + RS_STAGES, gw);
    }
    // the group leaves as one if a wait has run out (a thread of it samples the flag, everybody reads the sample after
    // the barrier); in the whole-tile form the barrier also says that every warp has drained the slot
    if ((tid & 255) == 0) fail_snap[grp][(i >> 1) & 1] = fail_flag;
    named_barrier(1 + grp, 256);
    if (fail_snap[grp][(i >> 1) & 1]) break;
    if (!PIECES && (tid & 255) == 0) refill(i + RS_STAGES);

    for (int i_t = 0; i_t < s.len; ++i_t) {
      const size_t ov = tok_off(a, s, hd, i_t, V);
      const float kq_reg = n_kq, eg = n_eg;
      float vv[4], bb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) vv[j] = n_v[j], bb[j] = n_b[j];
      if (i_t + 1 < s.len) fetch(i, i_t + 1); else fetch(i + 2, 0);
      float pq[4] = {0.f, 0.f, 0.f, 0.f}, pk[4] = {0.f, 0.f, 0.f, 0.f}, kq_part = 0.f;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float kv = __shfl_sync(0xffffffffu, kq_reg, r), qv = __shfl_sync(0xffffffffu, kq_reg, 16 + r);
        kq_part = fmaf(kv, qv, kq_part);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          S[r][j] *= eg;
          pk[j] = fmaf(S[r][j], kv, pk[j]);
          pq[j] = fmaf(S[r][j], qv, pq[j]);
        }
      }
      *reinterpret_cast<float4 *>(&sRed[par][0][gw][c0]) = make_float4(pq[0], pq[1], pq[2], pq[3]);
      *reinterpret_cast<float4 *>(&sRed[par][1][gw][c0]) = make_float4(pk[0], pk[1], pk[2], pk[3]);
      if (lane == 0) sKQ[par][gw] = kq_part;
      named_barrier(1 + grp, 256);
      float kq = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) pq[j] = pk[j] = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float4 x = *reinterpret_cast<const float4 *>(&sRed[par][0][w][c0]);
        const float4 y = *reinterpret_cast<const float4 *>(&sRed[par][1][w][c0]);
        pq[0] += x.x, pq[1] += x.y, pq[2] += x.z, pq[3] += x.w;
        pk[0] += y.x, pk[1] += y.y, pk[2] += y.z, pk[3] += y.w;
        kq += sKQ[par][w];
      }
      par ^= 1;
      float vn[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float u_ = vv[j] - pk[j];
        if (a.u && gw == 0) reinterpret_cast<T *>(a.u)[ov + c0 + j] = Num<T>::t(u_);
        vn[j] = u_ * bb[j];
        pq[j] = fmaf(vn[j], kq, pq[j]);
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const float kv = __shfl_sync(0xffffffffu, kq_reg, r);
#pragma unroll
        for (int j = 0; j < 4; ++j) S[r][j] = fmaf(kv, vn[j], S[r][j]);
      }
      if (gw == 0) {
        if (sizeof(T) == 2) {
          uint2 pkd;
          if (Num<T>::id == FLAB_BF16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(pq[0], pq[1]), hi = __floats2bfloat162_rn(pq[2], pq[3]);
            pkd.x = *reinterpret_cast<uint32_t *>(&lo), pkd.y = *reinterpret_cast<uint32_t *>(&hi);
          } else {
            __half2 lo = __floats2half2_rn(pq[0], pq[1]), hi = __floats2half2_rn(pq[2], pq[3]);
            pkd.x = *reinterpret_cast<uint32_t *>(&lo), pkd.y = *reinterpret_cast<uint32_t *>(&hi);
          }
          *reinterpret_cast<uint2 *>(reinterpret_cast<T *>(a.o) + ov + c0) = pkd;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) reinterpret_cast<T *>(a.o)[ov + c0 + j] = Num<T>::t(pq[j]);
        }
      }
    }
    if (ht) {
      float *dst = ht + (size_t)item * K * V;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const int kk = r0 + r;
        if (kk < K) {
          const float4 x = make_float4(S[r][0], S[r][1], S[r][2], S[r][3]);
          if (STREAM_ST) st_streaming(dst + (size_t)kk * V + c0, x);
          else *reinterpret_cast<float4 *>(dst + (size_t)kk * V + c0) = x;
        }
      }
    }
  }
}

// FLA_B200_DECODE_VARIANT (0..7, read once) selects the kernel's memory-path options for measurements; default 6
// (evict-first loads + streaming stores: 0.1025 ms per step of 256 x 16 tiles against 0.1087 without either)
static int decode_variant() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("FLA_B200_DECODE_VARIANT");
    v = (e && e[0] >= '0' && e[0] <= '7') ? e[0] - '0' : 6;
  }
  return v;
}

template <typename T, int VARIANT> static int launch_recurrent_stream_v(const flab_args *a, cudaStream_t stream) {
  const size_t smem = (size_t)RS_STAGES * 128 * RC_V * sizeof(float);
  auto kern = recurrent_stream_kernel<T, VARIANT>;
  if (int e = set_smem(kern, smem)) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_items = a->N * a->H;
  kern<<<n_items < sms ? n_items : sms, 512, smem, stream>>>(*a, n_items);
  return check_launch("recurrent_delta_fwd(stream)");
}

template <typename T> static int launch_recurrent_stream(const flab_args *a, cudaStream_t stream) {
  switch (decode_variant()) {
    case 0: return launch_recurrent_stream_v<T, 0>(a, stream);
    case 1: return launch_recurrent_stream_v<T, 1>(a, stream);
    case 2: return launch_recurrent_stream_v<T, 2>(a, stream);
    case 3: return launch_recurrent_stream_v<T, 3>(a, stream);
    case 4: return launch_recurrent_stream_v<T, 4>(a, stream);
    case 5: return launch_recurrent_stream_v<T, 5>(a, stream);
    case 6: return launch_recurrent_stream_v<T, 6>(a, stream);
    default: return launch_recurrent_stream_v<T, 7>(a, stream);
  }
}

template <typename T, bool DELTA> static int launch_recurrent_fwd(const flab_args *a, cudaStream_t stream) {
  if (DELTA && a->V == RC_V && a->K <= 128 && a->K % 4 == 0 && a->h0 && reinterpret_cast<uintptr_t>(a->h0) % 16 == 0 &&
      (!a->ht || reinterpret_cast<uintptr_t>(a->ht) % 16 == 0) && reinterpret_cast<uintptr_t>(a->o) % 8 == 0)
    return launch_recurrent_stream<T>(a, stream);
  dim3 grid(cdiv(a->V, RC_V), a->N * a->H);
  if (a->K <= 64) {
    recurrent_fwd_kernel<T, 4, DELTA><<<grid, RC_WARPS * 32, 0, stream>>>(*a);
  } else if (a->K <= 128) {
    recurrent_fwd_kernel<T, 8, DELTA><<<grid, RC_WARPS * 32, 0, stream>>>(*a);
  } else {
    recurrent_fwd_kernel<T, 16, DELTA><<<grid, RC_WARPS * 32, 0, stream>>>(*a);
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
  FLAB_REQUIRE(!a->ht || a->ht != a->h0 || (a->flags & FLAB_F_INPLACE_STATE), FLAB_E_BADARG,
               "recurrent_fwd: ht aliases h0; pass FLAB_F_INPLACE_STATE to update the state in place");
  FLAB_DISPATCH_ALL(a->dtype, T, return (launch_recurrent_fwd<T, false>(a, (cudaStream_t)stream)));
  return FLAB_OK;
}

int flab_recurrent_delta_fwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->o, FLAB_E_BADARG, "recurrent_delta_fwd needs q, k, v and o");
  FLAB_REQUIRE(!a->gk && !a->gv, FLAB_E_UNSUPPORTED, "recurrent_delta_fwd: only the scalar gate g is supported");
  FLAB_REQUIRE(a->K <= 256, FLAB_E_UNSUPPORTED, "recurrent_delta_fwd: K = %d > 256", a->K);
  // every (sequence, head, value slab) tile of the state is read in full by the one CTA that later writes it, so an
  // in-place update is safe; the caller has to say that it means it
  FLAB_REQUIRE(!a->ht || a->ht != a->h0 || (a->flags & FLAB_F_INPLACE_STATE), FLAB_E_BADARG,
               "recurrent_delta_fwd: ht aliases h0; pass FLAB_F_INPLACE_STATE to update the state in place");
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
