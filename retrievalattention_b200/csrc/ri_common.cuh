// Shared helpers for libri_b200: error reporting, 16-bit element traits, warp-level MMA.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "ri_b200.h"

// ---- error reporting (ri_error.cu) ---------------------------------------------------------
int ri_fail(int status, const char* fmt, ...);

#define RI_REQUIRE(cond, ...)                                  \
  do {                                                         \
    if (!(cond)) return ri_fail(RI_ERR_INVALID, __VA_ARGS__);  \
  } while (0)

#define RI_CUDA_OK(expr)                                                                   \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return ri_fail(RI_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                     __FILE__, __LINE__);                                                  \
  } while (0)

#define RI_LAUNCH_OK(name)                                                                        \
  do {                                                                                            \
    cudaError_t e__ = cudaGetLastError();                                                         \
    if (e__ != cudaSuccess)                                                                       \
      return ri_fail(RI_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__));      \
  } while (0)

static inline int64_t ri_align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }
__host__ __device__ constexpr size_t ri_align16(size_t x) { return (x + 15) & ~(size_t)15; }

// ---- 16-bit element traits -----------------------------------------------------------------
// DT = RI_BF16 (0) or RI_F16 (1).  Storage is 16 bits, all arithmetic accumulates in fp32.
template <int DT>
struct Elem;

template <>
struct Elem<RI_BF16> {
  __device__ __forceinline__ static float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  __device__ __forceinline__ static uint16_t bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
  __device__ __forceinline__ static float from_bits(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
  __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

template <>
struct Elem<RI_F16> {
  __device__ __forceinline__ static float round(float x) { return __half2float(__float2half_rn(x)); }
  __device__ __forceinline__ static uint16_t bits(float x) { return __half_as_ushort(__float2half_rn(x)); }
  __device__ __forceinline__ static float from_bits(uint16_t b) { return __half2float(__ushort_as_half(b)); }
  __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// Order-preserving map of a 16-bit float pattern onto uint16 (larger float -> larger key).
__device__ __forceinline__ uint16_t ri_ordered_key(uint16_t b) {
  return (b & 0x8000u) ? (uint16_t)~b : (uint16_t)(b | 0x8000u);
}

__device__ __forceinline__ uint4 ri_ldg16(const uint4* p) { return __ldg(p); }

constexpr float RI_LOG2E = 1.4426950408889634f;

// ---- programmatic dependent launch ------------------------------------------------------------
// Every kernel of the decode chain starts with ri_pdl_enter(): it lets the next kernel in the
// stream be scheduled right away (its CTAs become resident and run up to their own
// ri_pdl_enter) and then waits until the previous kernel has completed and its writes are
// visible.  All global reads and writes of a kernel come after this call, so the chain keeps
// plain stream-order semantics while the launch latency between dependent kernels is hidden.
// Launched without the attribute (or after a non-kernel operation) both instructions are no-ops.
// Measured on B200: worth a few tenths of a microsecond per launch for scan and select (ids 0, 1,
// on by default).  The attend kernel (id 2: 8-CTA clusters with ~100 KB of shared memory each)
// got slower when its CTAs became resident early, so it and the steady append (id 4) are
// launched in plain stream order.  The single decode kernel (id 5) and the gather wait (id 6) are
// on: on one GPU it makes no difference to the decode kernel, between several GPUs the wait
// kernel's launch hides behind the decode kernel and the next decode kernel's behind the wait.
// The element-wise kernels of the decode layer (id 8) are on: their launch hides behind the library GEMM
// in front of them (measured: 2 % of the whole model step).
__device__ __forceinline__ void ri_pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t ri_launch_pdl_id(int id, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  static const int mask = getenv("RI_PDL_MASK") ? atoi(getenv("RI_PDL_MASK")) : 0x163;   // per-kernel switch
  cfg.attrs = attr;
  cfg.numAttrs = (mask >> id) & 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
