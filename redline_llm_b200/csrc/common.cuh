// Shared helpers of the sm_100a decode kernels: status plumbing for the C ABI,
// per-device facts cached on first use, 128-bit access helpers.
#pragma once

#include <cstdint>
#include <cstdio>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/redline_kernels.h"

namespace rl {

constexpr int kKvBlock = 16;  // tokens per KV page (src/core/types.hpp: kKvBlockSize)
constexpr int kKvBlockShift = 4;

// Records `msg` for rl_last_error() and returns `code`.
int Fail(int code, const char* fmt, ...);

// cudaGetLastError() after a launch, folded into the ABI's status convention.
int LaunchStatus(const char* what);

struct DeviceFacts {
  int sm_count = 0;
  int max_smem_optin = 0;
  bool ready = false;
};
// Facts of the CURRENT device, queried once per device (first call happens in
// warm-up, outside any stream capture) and a plain array read afterwards.
const DeviceFacts& CurrentDeviceFacts();
int CurrentDeviceIndex();

// Process-wide opt-in (rl_attention_set_prologue_overlap): launch the decode-sized kernels with
// programmatic stream serialisation. Kernels launched this way start with griddepcontrol.wait (the
// attention kernel after its table walk), so they never read or write before the previous kernel of
// the stream has completed; what overlaps is the launch itself and, for attention, the walk.
extern bool g_launch_overlap;

template <typename... KArgs, typename... Args>
inline cudaError_t LaunchOverlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_launch_overlap ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// First statement of a kernel that may be launched by LaunchOverlapped: let the next such launch
// be set up now, then wait for the previous kernel of the stream (a no-op for ordinary launches).
__device__ __forceinline__ void DependentLaunchGate() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// First-use set-up of the decode linear kernel on the current device (shared-memory opt-in, driver
// entry point, error flag); rl_kernels_init calls it so that no launcher does set-up inside a capture.
int DecodeLinearInit();

inline bool Aligned16(const void* p) { return (reinterpret_cast<std::uintptr_t>(p) & 15u) == 0; }

// 16-byte global access. .nc loads are for data this kernel never writes.
__device__ __forceinline__ uint4 LdgStream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 Ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void Stg16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ half2 AsHalf2(uint32_t u) { return *reinterpret_cast<half2*>(&u); }
__device__ __forceinline__ uint32_t AsU32(half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

}  // namespace rl
