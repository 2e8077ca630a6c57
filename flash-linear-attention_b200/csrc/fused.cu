// Whole-forward entry points of chunk_gated_delta_rule: cumsum -> WY -> state scan -> output as one
// C call (four kernel launches, no host work in between).  Intermediates (cumsummed gate, Aw, Au, w, u,
// chunk states, v_new) live in caller-provided scratch memory.
// Stage order follows chunk_gated_delta_rule_fwd (fla/ops/gated_delta_rule/chunk.py:20-73).
#include "common.cuh"

extern "C" size_t flab_gated_delta_rule_fwd_workspace(const flab_args *a);

namespace flab {

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

struct FwdScratch {
  size_t g, aw, au, w, u, h, v_new, total;
};

static FwdScratch scratch_layout(const flab_args *a) {
  const size_t tok = (size_t)a->B * a->T * a->H, e = 2;
  FwdScratch s;
  size_t off = 0;
  s.g = off, off += align256(tok * sizeof(float));
  s.aw = off, off += align256(tok * C * e);
  s.au = off, off += align256(tok * C * e);
  s.w = off, off += align256(tok * a->K * e);
  s.u = off, off += align256(tok * a->V * e);
  s.v_new = off, off += align256(tok * a->V * e);
  s.h = off, off += align256((size_t)a->NT * a->H * a->K * a->V * e);
  s.total = off;
  return s;
}

static int run_fwd(const flab_args *a, unsigned char *ws, void *stream) {
  const FwdScratch L = scratch_layout(a);
  flab_args s = *a;
  s.ws = nullptr;
  s.ws_bytes = 0;
  // 1. chunk-local cumsum of the raw gate (fp32 in, fp32 out)
  flab_args c = s;
  c.dtype = FLAB_FP32;
  c.flags = 0;
  c.x = a->g;
  c.y = ws + L.g;
  if (int e = flab_chunk_local_cumsum_scalar(&c, stream)) return e;
  s.g = ws + L.g;
  // 2. WY factors
  s.aw = ws + L.aw, s.au = ws + L.au, s.w = ws + L.w, s.u = ws + L.u;
  if (int e = flab_wy_fwd(&s, stream)) return e;
  // 3. state scan
  s.h = ws + L.h, s.v_new = ws + L.v_new;
  if (int e = flab_delta_fwd_h(&s, stream)) return e;
  // 4. output (v := v_new)
  flab_args o = s;
  o.v = ws + L.v_new;
  return flab_chunk_fwd_o(&o, stream);
}

static int check_fwd_args(const flab_args *a, const char *who) {
  if (int e = check_common(a)) return e;
  FLAB_REQUIRE(a->q && a->k && a->v && a->g && a->beta && a->o, FLAB_E_BADARG, "%s needs q, k, v, g, beta and o", who);
  FLAB_REQUIRE(a->dtype == FLAB_BF16 || a->dtype == FLAB_FP16, FLAB_E_UNSUPPORTED, "%s: bf16 / fp16 only", who);
  FLAB_REQUIRE(a->NT > 0, FLAB_E_BADARG, "%s: NT must be positive", who);
  return 0;
}

}  // namespace flab

extern "C" {

size_t flab_gated_delta_rule_fwd_workspace(const flab_args *a) {
  if (!a || a->B <= 0 || a->T <= 0 || a->H <= 0 || a->NT <= 0) return 0;
  return flab::scratch_layout(a).total;
}

int flab_gated_delta_rule_fwd(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_fwd_args(a, "gated_delta_rule_fwd")) return e;
  const size_t need = scratch_layout(a).total;
  FLAB_REQUIRE(a->ws && a->ws_bytes >= need, FLAB_E_BADARG, "gated_delta_rule_fwd: workspace of %zu bytes needed, %zu given",
               need, a->ws_bytes);
  FLAB_REQUIRE(reinterpret_cast<uintptr_t>(a->ws) % 256 == 0, FLAB_E_BADARG, "gated_delta_rule_fwd: workspace must be 256-byte aligned");
  return run_fwd(a, static_cast<unsigned char *>(a->ws), stream);
}

}
