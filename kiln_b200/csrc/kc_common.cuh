// Shared device helpers for the kiln-cuda kernels (sm_100a only).
//
// Everything that waits on the device (mbarrier phases) is bounded: a wait
// that does not complete within KC_SPIN_LIMIT_NS records a code in the
// context's status word and returns false, so a broken pipeline ends as an
// error status on the host instead of a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

#ifndef __CUDA_ARCH_FEAT_SM100_ALL
#if defined(__CUDA_ARCH__)
#error "kiln-cuda kernels are written for sm_100a only (compile with -gencode arch=compute_100a,code=sm_100a)"
#endif
#endif

namespace kc {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// Status word codes: (kernel id << 8) | wait id.
enum : uint32_t {
  KC_DEV_QLINEAR = 0x100,
  KC_DEV_ATTN = 0x200,
  KC_DEV_TP = 0x300,
};

constexpr unsigned long long KC_SPIN_LIMIT_NS = 1500ull * 1000ull * 1000ull;  // 1.5 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ----------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// One try_wait: the thread may be suspended by the hardware until the phase completes or the hinted time
// (nanoseconds) has passed, so a waiting warp does not burn issue slots spinning.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded busy-poll (no hardware suspend): lowest wake-up latency, costs issue slots.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t code) {
  if (mbar_test_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_test_wait(bar, parity)) {
    if ((++spins & 0xfff) == 0) {
      if (globaltimer_ns() - t0 > KC_SPIN_LIMIT_NS) {
        if (status) atomicOr(status, code);
        return false;
      }
    }
  }
  return true;
}
// Bounded wait. On timeout: ORs `code` into *status (if non-null) and returns
// false; the caller must then leave its pipeline loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* status,
                                          uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3f) == 0) {
      if (globaltimer_ns() - t0 > KC_SPIN_LIMIT_NS) {
        if (status) atomicOr(status, code);
        return false;
      }
    }
  }
  return true;
}

// ---- async-proxy fences, bulk copies (TMA) --------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// 2-D tiled TMA load (no multicast): coordinates {x = innermost, y}.
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int32_t x,
                                            int32_t y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 4-D tiled TMA load (no multicast): coordinates {x = innermost, y, z, w}; x * element size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, int32_t x, int32_t y, int32_t z,
                                            int32_t w, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- bf16 helpers --------------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
  bf162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf162(uint32_t u) {
  bf162 v = *reinterpret_cast<bf162*>(&u);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- programmatic dependent launch ---------------------------------------
// Every kernel of the step is launched with programmatic stream serialization: it may become resident while
// its predecessor in the stream is still running, executes whatever touches no step data (barrier set-up,
// TMEM allocation, descriptor prefetch, loads of WEIGHTS, which no kernel writes), and calls pdl_wait() before
// its first access to memory that an earlier kernel of the stream writes or reads. pdl_wait() returns once the
// predecessor grid has completed and its writes are visible; since every kernel calls it before it ends, a
// kernel's completion implies the completion of everything queued before it. pdl_launch_dependents() lets the
// successor start being scheduled; it is issued first thing, so the successor fills SMs as they drain.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// One-time set-up that has to happen once per DEVICE (kernel attributes live in the device's copy of the module, and
// one process may hold contexts on several devices). Host threads of different contexts may race here: the worst
// case is that the set-up runs twice, which is harmless.
struct DeviceOnce {
  unsigned long long done = 0;   // bit d: device d is configured (devices past 63 are configured on every call)
  bool first_on_current_device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d > 63) return true;
    if (done >> d & 1ull) return false;
    done |= 1ull << d;
    return true;
  }
  void forget_current_device() {
    int d = 0;
    if (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d <= 63) done &= ~(1ull << d);
  }
};

// allow_early = false launches with plain stream order: used for the first kernel after a collective, whose duration
// depends on the OTHER ranks — nothing of this library may be resident and counting down a bounded wait meanwhile.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k_opt(bool allow_early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (allow_early) { cfg.attrs = attr; cfg.numAttrs = 1; }
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  return launch_k_opt(true, kernel, grid, block, smem, s, std::forward<Args>(args)...);
}

// Mlp::forward activation (nn.rs:284-294): silu(gate) * up with the three bf16 roundings of the composed ops, or
// gelu_approx(gate) * up op for op (nn.rs:221-235). g and u are bf16 values held in fp32; so is the result.
__device__ __forceinline__ float act_silu_mul(float g, float u) {
  const float s = bf16_round(1.f / (1.f + __expf(-g)));
  const float t = bf16_round(g * s);
  return bf16_round(t * u);
}
__device__ __forceinline__ float act_gelu_mul(float g, float u) {
  const float cube = bf16_round(g * g * g);  // power(x, 3) in fp32, rounded once
  const float inner = bf16_round(g + bf16_round(bf16_round(0.044715f) * cube));
  const float scaled = bf16_round(bf16_round(0.7978845608028654f) * inner);
  const float gate = bf16_round(1.f + bf16_round(tanhf(scaled)));
  const float act = bf16_round(bf16_round(0.5f * g) * gate);
  return bf16_round(act * u);
}

// A ring position: stage index and phase bit, advanced without division.
struct RingPos {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n_stages) {
    if (++stage == n_stages) { stage = 0; phase ^= 1u; }
  }
};

}  // namespace kc
