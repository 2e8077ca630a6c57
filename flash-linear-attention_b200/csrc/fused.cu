// Whole-forward entry points of chunk_gated_delta_rule: cumsum -> WY -> state scan -> output as one
// C call (four kernel launches, no host work in between).  Intermediates (cumsummed gate, Aw, Au, w, u,
// chunk states, v_new) live in scratch memory: caller-provided for flab_gated_delta_rule_fwd, a
// file-scope device array for flab_gated_delta_rule_fwd_noalloc.
// Stage order follows chunk_gated_delta_rule_fwd (fla/ops/gated_delta_rule/chunk.py:20-73).
#include <mutex>

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

// ---- scratch that nobody allocates -----------------------------------------------------------------
// 16 MiB per GPU that loads the library, held until the process exits.  It covers B*T*H <= 8192
// token-heads at K = V = 128 (for example one 512-token prompt of a 16-head layer).
constexpr size_t NOALLOC_BYTES = 16u << 20;
static __device__ __align__(256) unsigned char g_fwd_scratch[NOALLOC_BYTES];

// In host code `g_fwd_scratch` is only a stand-in for the device array: its device address has to be
// asked for, once per device, with that device current.
static std::mutex g_scratch_mutex;
static unsigned char *g_scratch_ptr[64] = {nullptr};

static int scratch_device_pointer(unsigned char **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  FLAB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, FLAB_E_LAUNCH, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_fwd_scratch);
    FLAB_REQUIRE(e == cudaSuccess && p != nullptr, FLAB_E_LAUNCH, "cudaGetSymbolAddress(g_fwd_scratch) failed: %s",
                 cudaGetErrorString(e));
    g_scratch_ptr[dev] = static_cast<unsigned char *>(p);
  }
  *out = g_scratch_ptr[dev];
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

int flab_gated_delta_rule_fwd_noalloc(const flab_args *a, void *stream) {
  using namespace flab;
  if (int e = check_fwd_args(a, "gated_delta_rule_fwd_noalloc")) return e;
  const size_t need = scratch_layout(a).total;
  FLAB_REQUIRE(need <= NOALLOC_BYTES, FLAB_E_UNSUPPORTED,
               "gated_delta_rule_fwd_noalloc: this problem needs %zu bytes of scratch, the built-in scratch holds %zu "
               "(B*T*H <= 8192 at K = V = 128); use flab_gated_delta_rule_fwd with a caller workspace",
               need, (size_t)NOALLOC_BYTES);
  unsigned char *ws = nullptr;
  if (int e = scratch_device_pointer(&ws)) return e;
  return run_fwd(a, ws, stream);
}
}
