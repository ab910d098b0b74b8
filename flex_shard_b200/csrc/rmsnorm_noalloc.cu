// RMSNorm backward without any allocation: the weight-gradient partial sums go through a fixed
// array that is part of the library image. See fsb_noalloc.h for who needs this and for the rules
// (size limit, first call before stream capture, no overlapping calls).
#include "common.cuh"
#include "fsb_noalloc.h"
#include <stdio.h>

namespace {
using namespace fsb;

constexpr long long kScratchFloats = 2LL * 1024 * 1024;  // 8 MiB, resident on every GPU that loads the library
constexpr int kThreads = 256;
constexpr int kRowsPerBlock = 32;
constexpr int kMaxDevices = 64;

// File-scope device array. In host code this name is only a handle for the runtime, not a device
// address: the address is looked up once per device below and handed to the kernels.
static __device__ __align__(256) float g_dw_scratch[kScratchFloats];

float* g_scratch_addr[kMaxDevices] = {nullptr};

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(t.v[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < kThreads / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// One CTA per 32 rows: per row dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres) with xhat = x*rstd, and the
// CTA's sum of dy*xhat over its rows goes to one fp32 row of `partial` (here: the built-in array). The
// ordinary entry point computes the same quantities with a different thread layout, so the two agree to
// rounding, not bit for bit.
__global__ void __launch_bounds__(kThreads)
rmsnorm_bwd_noalloc_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                           const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                           float* __restrict__ partial, long long T, int D) {
  __shared__ float red[32];
  float dwacc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[a][j] = 0.f;
  const long long row0 = static_cast<long long>(blockIdx.x) * kRowsPerBlock;
  for (int rr = 0; rr < kRowsPerBlock; ++rr) {
    const long long row = row0 + rr;
    if (row >= T) break;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = threadIdx.x * 8; i < D; i += kThreads * 8) {
      float a[8], b[8], c[8];
      load8(dy + row * D + i, a);
      load8(x + row * D + i, b);
      load8(w + i, c);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * c[j] * b[j];
    }
    dot = block_sum(dot, red);
    const float coef = dot * r * r * r / D;
    int g = 0;
    for (int i = threadIdx.x * 8; i < D; i += kThreads * 8, ++g) {
      float a[8], b[8], c[8], o[8];
      load8(dy + row * D + i, a);
      load8(x + row * D + i, b);
      load8(w + i, c);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = a[j] * c[j] * r - b[j] * coef;
        if (g < 4) dwacc[g][j] += a[j] * b[j] * r;
      }
      if (dres) {
        float e[8];
        load8(dres + row * D + i, e);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += e[j];
      }
      store8(dx + row * D + i, o);
    }
  }
  int g = 0;
  for (int i = threadIdx.x * 8; i < D; i += kThreads * 8, ++g) {
    if (g < 4) {
      float* p = partial + static_cast<long long>(blockIdx.x) * D + i;
      *reinterpret_cast<float4*>(p) = make_float4(dwacc[g][0], dwacc[g][1], dwacc[g][2], dwacc[g][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dwacc[g][4], dwacc[g][5], dwacc[g][6], dwacc[g][7]);
    }
  }
}

// Column sums of the partial rows in block order (deterministic).
__global__ void colsum_noalloc_kernel(const float* __restrict__ partial, void* __restrict__ out, int P, int D,
                                      int out_fp32, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[static_cast<long long>(p) * D + c];
  if (out_fp32) {
    float* o = static_cast<float*>(out);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

}  // namespace

extern "C" __attribute__((visibility("default"))) long long fsb_rmsnorm_bwd_noalloc_capacity(void) {
  return kScratchFloats;
}

extern "C" __attribute__((visibility("default"))) int
fsb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                        void* dx, void* dw_out, int dw_fp32, int dw_accumulate, long long T, int D,
                        cudaStream_t stream) {
  if (D <= 0 || D % 8 != 0 || D > 8192 || T <= 0) return FSB_ERR_BAD_ARG;
  const long long blocks = (T + kRowsPerBlock - 1) / kRowsPerBlock;
  if (blocks * D > kScratchFloats) {
    fprintf(stderr,
            "[fsb200] fsb_rmsnorm_bwd_noalloc: T=%lld, D=%d needs %lld scratch floats, the built-in array "
            "holds %lld; use fsb_rmsnorm_bwd with a caller-provided buffer for this size\n",
            T, D, blocks * D, kScratchFloats);
    return FSB_ERR_TOO_LARGE;
  }
  // the kernels use 16-byte accesses on the bf16 tensors and element accesses on rstd / dw_out: a null or
  // misaligned pointer is refused here instead of faulting on the device
  const auto misaligned = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr || dw_out == nullptr)
    return FSB_ERR_BAD_ARG;
  if (misaligned(dy, 16) || misaligned(x, 16) || misaligned(w, 16) || misaligned(dx, 16) ||
      (dres != nullptr && misaligned(dres, 16)) || misaligned(rstd, 4) || misaligned(dw_out, dw_fp32 ? 4 : 2))
    return FSB_ERR_BAD_ARG;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FSB_ERR_LAUNCH;
  if (g_scratch_addr[dev] == nullptr) {
    // set-up, once per device, with that device current: the array's address on THIS device
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_dw_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "[fsb200] fsb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      return FSB_ERR_LAUNCH;
    }
    g_scratch_addr[dev] = ptr;
  }
  float* scratch = g_scratch_addr[dev];
  rmsnorm_bwd_noalloc_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),
      static_cast<__nv_bfloat16*>(dx), scratch, T, D);
  if (cudaGetLastError() != cudaSuccess) return FSB_ERR_LAUNCH;   // the second launch would read an unwritten array
  colsum_noalloc_kernel<<<(D + 255) / 256, 256, 0, stream>>>(scratch, dw_out, static_cast<int>(blocks), D,
                                                              dw_fp32, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
