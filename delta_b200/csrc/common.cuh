// Shared helpers of the hand-written sm_100a kernels.
//
// Every launcher in this library has C linkage, takes raw device pointers and a
// stream, allocates nothing, and returns 0 or a negative code; the text of the
// last refusal is kept for dk_last_error().  Tensors are addressed by element
// type code: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define DK_F32 0
#define DK_BF16 1

#define DK_ERR_ARG (-1)
#define DK_ERR_LAUNCH (-2)

extern "C" const char* dk_last_error();
void dk_set_error(const char* fmt, ...);

#define DK_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      dk_set_error(__VA_ARGS__);         \
      return DK_ERR_ARG;                 \
    }                                    \
  } while (0)

// What a launcher has asked of a device (its number of SMs, the dynamic shared memory a kernel was granted there)
// is kept per device: the answers of one device say nothing about another.
constexpr int DK_MAX_DEVICES = 64;
static inline int dk_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
  return dev % DK_MAX_DEVICES;
}
static inline int dk_sm_count() {
  static int sms[DK_MAX_DEVICES] = {0};
  const int dev = dk_current_device();
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

static inline int dk_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    dk_set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return DK_ERR_LAUNCH;
  }
  return 0;
}

// Device-side record of a bad index: kernels that follow page tables check what
// they read, write {code, a, b, c} once and skip the access, so that a wrong
// table shows up as an error on the host and not as a memory fault.
#define DK_DEV_BAD_PAGE 1
#define DK_DEV_BAD_TOKEN 2
#define DK_DEV_BAD_POSITION 3

__device__ __forceinline__ void dk_report(int* err, int code, int a, int b, int c) {
  if (err != nullptr && atomicCAS(err, 0, code) == 0) {
    err[1] = a;
    err[2] = b;
    err[3] = c;
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
