// Shared helpers of the tpx_b200 CUDA library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/tpx_b200.h"

namespace tpx {

// Thread-local error text behind tpx_last_error().
void set_error(const char* fmt, ...);

#define TPX_REQUIRE(cond, code, ...)      \
  do {                                    \
    if (!(cond)) {                        \
      ::tpx::set_error(__VA_ARGS__);      \
      return (code);                      \
    }                                     \
  } while (0)

#define TPX_CUDA_OK(call)                                                                  \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      ::tpx::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return TPX_ERR_CUDA;                                                                 \
    }                                                                                      \
  } while (0)

#define TPX_LAUNCH_OK()                                                                    \
  do {                                                                                     \
    cudaError_t e__ = cudaGetLastError();                                                  \
    if (e__ != cudaSuccess) {                                                              \
      ::tpx::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__), __FILE__, __LINE__); \
      return TPX_ERR_CUDA;                                                                 \
    }                                                                                      \
  } while (0)

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }

// fp32 -> bf16 bits, round to nearest even (matches at::BFloat16 and the CPU oracle)
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case TPX_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    case TPX_ACT_SILU: return v / (1.0f + __expf(-v));
    case TPX_ACT_RELU: return fmaxf(v, 0.0f);
    default: return v;
  }
}

int sm_count();
void count_launch();  // host-side tally behind tpx_launch_count()

// Kernel-selection switches, read from the environment once (first use) and again on tpx_reload_options():
// TPX_TC_WHOLE, TPX_TC_WIDE, TPX_TC_F4, TPX_TC_W4 (-1 = let the planner decide), TPX_TC_CLUSTER (0 = no cluster split-K),
// TPX_TC_PF (L2 prefetch distance), TPX_HANDOFF_MIN_TOKENS (fewest tokens at which gate/up hands its output to down as terms), TPX_ATTN_SPLITS (0 = cost model), TPX_ATTN_TC (0 = prefill attention on the mma.sync kernel). None of them changes a result. `dbg` carries
// TPX_TC_DBG and is always 0 unless the library was built with -DTPX_DEBUG.
struct Knobs {
  int tc_whole, tc_wide, tc_f4, tc_w4, tc4_occ, tc_cluster, tc_pf, handoff_min, tc_p, tc_p2, tc_p_uks, tc_p_rows, attn_splits, attn_tc, dbg;
};
const Knobs& knobs();

// Programmatic dependent launch. Every kernel of the decoder-layer path starts with pdl_trigger() (the next
// kernel in the stream may be scheduled and run its prologue while this one works) and calls pdl_wait() before
// it touches global memory that an earlier kernel may have written or may still read: the wait returns once
// every earlier grid has completed and its writes are visible, so the memory order is that of plain stream
// launches and only launch latency and prologues overlap.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tpx
