// Shared device/host helpers for the dartkv_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dartkv_b200.h"

// ---------------------------------------------------------------------------- errors
void dartkv_set_error(const char* fmt, ...);
void dartkv_count_launch();

#define DARTKV_REQUIRE(cond, ...)          \
  do {                                     \
    if (!(cond)) {                         \
      dartkv_set_error(__VA_ARGS__);       \
      return DARTKV_EINVAL;                \
    }                                      \
  } while (0)

#define DARTKV_CUDA_OK(expr)                                                        \
  do {                                                                              \
    cudaError_t err__ = (expr);                                                     \
    if (err__ != cudaSuccess) {                                                     \
      dartkv_set_error("%s failed: %s", #expr, cudaGetErrorString(err__));          \
      return DARTKV_ECUDA;                                                          \
    }                                                                               \
  } while (0)

#define DARTKV_LAUNCH_OK(name)                                                      \
  do {                                                                              \
    cudaError_t err__ = cudaGetLastError();                                         \
    if (err__ != cudaSuccess) {                                                     \
      dartkv_set_error("launch of %s failed: %s", name, cudaGetErrorString(err__)); \
      return DARTKV_ECUDA;                                                          \
    }                                                                               \
    dartkv_count_launch();                                                          \
  } while (0)

static inline bool dartkv_valid_dtype(int dt) { return dt == DARTKV_F32 || dt == DARTKV_F16 || dt == DARTKV_BF16; }
__host__ __device__ __forceinline__ int dartkv_dtype_size(int dt) { return dt == DARTKV_F32 ? 4 : 2; }
static inline int dartkv_dtype_bytes(int dt) { return dt == DARTKV_F32 ? 4 : 2; }
static inline bool dartkv_valid_bits(int bits) { return bits == 2 || bits == 4 || bits == 8; }

// ---------------------------------------------------------------------------- rounding model
// The reference evaluates each elementwise op of a bf16/fp16 tensor in fp32 and rounds the
// result back to the tensor dtype; rnd() is that rounding.  __fadd_rn/__fmul_rn/__fdiv_rn keep
// the compiler from contracting separately-rounded steps into an fma.
__device__ __forceinline__ float rnd_rt(float x, int dt) {
  if (dt == DARTKV_F16) return __half2float(__float2half_rn(x));
  if (dt == DARTKV_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

template <int DT>
__device__ __forceinline__ float rnd(float x) {
  if (DT == DARTKV_F16) return __half2float(__float2half_rn(x));
  if (DT == DARTKV_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

__device__ __forceinline__ float load_f(const void* p, int dt, int64_t i) {
  if (dt == DARTKV_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  if (dt == DARTKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

// value must already be representable in dt (or the caller wants round-to-nearest-even)
__device__ __forceinline__ void store_f(void* p, int dt, int64_t i, float v) {
  if (dt == DARTKV_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else if (dt == DARTKV_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

__device__ __forceinline__ float quant_eps(int dt) { return dt == DARTKV_F32 ? 1e-6f : rnd_rt(1e-4f, dt); }

// scale of a group: clamp(max - min, eps) / qmax, every step rounded to the data dtype
__device__ __forceinline__ float group_scale(float mn, float mx, float qmax, int dt, int div_mode) {
  float range = rnd_rt(__fsub_rn(mx, mn), dt);
  range = fmaxf(range, quant_eps(dt));
  if (div_mode == DARTKV_DIV_RECIPROCAL) return rnd_rt(__fmul_rn(range, __fdiv_rn(1.0f, qmax)), dt);
  return rnd_rt(__fdiv_rn(range, qmax), dt);
}

// code of one element: clamp(rint(rnd(rnd(x - min) / scale)), 0, qmax)
__device__ __forceinline__ uint32_t group_code(float x, float mn, float scale, float qmax, int dt) {
  float shifted = rnd_rt(__fsub_rn(x, mn), dt);
  float ratio = rnd_rt(__fdiv_rn(shifted, scale), dt);
  float q = fminf(fmaxf(rintf(ratio), 0.0f), qmax);
  return (uint32_t)q;
}

// dequantized element in the output dtype, as float
__device__ __forceinline__ float affine_restore(float code, float scale, float zero, int md, int out_dt, int flavour) {
  float v;
  if (flavour == DARTKV_DEQUANT_FUSED) return __fmaf_rn(code, scale, zero);   // attention-only: nothing is rounded
  if (flavour == DARTKV_DEQUANT_FP32) {
    v = __fmaf_rn(code, scale, zero);
  } else {
    v = rnd_rt(__fadd_rn(rnd_rt(__fmul_rn(code, scale), md), zero), md);
  }
  return rnd_rt(v, out_dt);
}

__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Balanced split of `units` work units over `blocks` blocks: block j owns [j*units/blocks, (j+1)*units/blocks).
// Returns the block that owns unit x.
__host__ __device__ __forceinline__ int dartkv_block_of_unit(int64_t x, int blocks, int64_t units) {
  int64_t j = x * blocks / units;
  if ((j + 1) * units / blocks <= x) ++j;
  return (int)j;
}

static inline int dartkv_gcd(int a, int b) { while (b) { int t = a % b; a = b; b = t; } return a; }
