// Views of the opaque C-ABI handles for entry points that live outside kc_api.cu. The handle structs stay
// private to kc_api.cu; these accessors (defined there) hand out only what another translation unit needs.
#pragma once

#include "kc_qlinear.cuh"

struct kc_ctx;
struct kc_qweight;

namespace kc {

struct CtxView {
  int device;
  cudaStream_t stream;
  uint32_t* status;  // device status word of the context
};

CtxView ctx_view(kc_ctx* c);
const QWeight* qweight_view(kc_qweight* q);
kc_ctx* qweight_owner(kc_qweight* q);   // the context the weight's device memory belongs to
// Adds n launches of the GEMM (cls 0) / split-K reduction (cls 1) class to the context's launch counters.
void ctx_count_launches(kc_ctx* c, int cls, int n);
// Records `msg` as the calling thread's last error (what kc_last_error returns) and returns `code`.
int api_fail(int code, const char* msg);

}  // namespace kc
