// kc_quantized_matmul_static: the affine-quantised matmul of kc_quantized_matmul with its split-K workspace in a
// fixed device array of this library instead of an allocation owned by the weight handle.
//
// kc_quantized_matmul reads its fp32 split-K partials from a buffer that kc_qweight_create sized with cudaMalloc
// (splits x 512 rows x out_features). This entry point makes no device or pinned-host allocation at all — no
// cudaMalloc / cudaFree, no stream-ordered allocation, nothing that can call them — so it can be used where an
// allocation is not permitted or not affordable: between other people's kernels on a stream whose memory pool the
// caller does not own, in a latency-critical loop where a cudaMalloc would serialise the device, or with the
// device's memory already handed out to the last byte. The workspace is the file-scope array below; it is part of
// the library image and is placed on each device when the library's module is loaded there.
//
// Limits and behaviour a caller must know:
//   * the partials of one launch (splits x min(m, 512) x out_features fp32) must fit KC_STATIC_SCRATCH_BYTES
//     (16 MiB); a larger request is rejected with KC_ERR_UNSUPPORTED before anything is launched. Weights that are
//     not split along K use no scratch and are never rejected for size;
//   * the first call on a device resolves the array's address (cudaGetSymbolAddress, which loads the module on
//     that device if it is not loaded yet) and creates the kernel's attributes; make that first call before any
//     stream capture begins;
//   * the array is shared by every context and every weight on the device and keeps whatever the last call left in
//     it. Calls that overlap in time on the same device (two streams, two threads) race on it: serialise them.
//
// The kernels, their launch geometry and the order of the fp32 additions are those of kc_quantized_matmul, so the
// two entry points return the same bits.
#include "../../include/kiln_cuda.h"

#include <cstdio>

#include "kc_internal.cuh"

using namespace kc;

#define KC_STATIC_SCRATCH_BYTES (16u << 20)

static __device__ __align__(256) unsigned char g_static_scratch[KC_STATIC_SCRATCH_BYTES];

extern "C" int64_t kc_static_scratch_bytes(void) { return (int64_t)KC_STATIC_SCRATCH_BYTES; }

extern "C" int kc_quantized_matmul_static(kc_ctx_t c, kc_qweight_t q, const void* x_dev, int32_t m, void* y_dev) {
  char msg[256];
  if (!c || !q || !x_dev || !y_dev) return api_fail(KC_ERR_INVALID, "kc_quantized_matmul_static: NULL argument");
  if (m < 1) {
    snprintf(msg, sizeof msg, "kc_quantized_matmul_static: m = %d", m);
    return api_fail(KC_ERR_INVALID, msg);
  }
  if ((uintptr_t)x_dev % 16) return api_fail(KC_ERR_INVALID, "kc_quantized_matmul_static: x must be 16-byte aligned");
  if (qweight_owner(q) != c)
    return api_fail(KC_ERR_INVALID, "kc_quantized_matmul_static: the weight was created on another context");
  const CtxView cv = ctx_view(c);
  const QWeight& w = *qweight_view(q);

  // Size check first: nothing is launched for a request the array cannot hold.
  const int slab = m < QL_MAX_M ? m : QL_MAX_M;
  const size_t need = w.splits > 1 ? (size_t)w.splits * slab * w.N * sizeof(float) : 0;
  if (need > KC_STATIC_SCRATCH_BYTES) {
    snprintf(msg, sizeof msg,
             "kc_quantized_matmul_static: %d splits x %d rows x %d features of fp32 partials = %zu bytes exceed the "
             "static scratch of %u bytes; use fewer rows per call or kc_quantized_matmul",
             w.splits, slab, w.N, need, KC_STATIC_SCRATCH_BYTES);
    return api_fail(KC_ERR_UNSUPPORTED, msg);
  }

  cudaError_t e = cudaSetDevice(cv.device);
  if (e != cudaSuccess) return api_fail(KC_ERR_CUDA, cudaGetErrorString(e));
  // Address of the array on the current device: resolved on every call, no state of this file depends on which
  // device called last.
  float* scratch = nullptr;
  e = cudaGetSymbolAddress((void**)&scratch, g_static_scratch);
  if (e != cudaSuccess || !scratch) {
    snprintf(msg, sizeof msg, "kc_quantized_matmul_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    return api_fail(KC_ERR_CUDA, msg);
  }

  // Tensor maps of the activation buffer live on this stack frame; the launch copies them into the kernel's
  // parameters. x must be readable for round_up(m, 16) rows, like kc_quantized_matmul.
  ActOperand op;
  const char* terr = "";
  if (!act_operand_init(&op, (const bf16*)x_dev, (m + 15) & ~15, w.K, &terr)) {
    snprintf(msg, sizeof msg, "kc_quantized_matmul_static: %s", terr);
    return api_fail(KC_ERR_CUDA, msg);
  }
  bf16* y = (bf16*)y_dev;
  for (int row0 = 0; row0 < m; row0 += QL_MAX_M) {
    QLinearLaunch l;
    l.w = &w; l.x = &op; l.row0 = row0; l.M = (m - row0) < QL_MAX_M ? (m - row0) : QL_MAX_M;
    l.y = y; l.ldy = w.N; l.partial = scratch; l.status = cv.status;
    // launches are counted once they are queued; this entry point takes no part in kc_profile_* timing
    e = qlinear_umma(l, cv.stream);
    if (e == cudaSuccess) ctx_count_launches(c, 0, qlinear_launches(w, l.M));
    if (e == cudaSuccess && w.splits > 1) {
      e = qlinear_reduce_splits(scratch, w.splits, l.M, w.N, y + (size_t)row0 * w.N, w.N, cv.stream);
      if (e == cudaSuccess) ctx_count_launches(c, 1, 1);
    }
    if (e != cudaSuccess) {
      snprintf(msg, sizeof msg, "kc_quantized_matmul_static: launch: %s", cudaGetErrorString(e));
      return api_fail(KC_ERR_CUDA, msg);
    }
  }
  return KC_OK;
}
