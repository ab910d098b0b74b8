// Muon's elementwise passes around the Newton-Schulz GEMMs (which run on gemm_bf16.cu):
//   prepare : M <- lerp(M, g, 1-mu); u = nesterov ? lerp(g, M, mu) : M; write u as bf16 and
//             accumulate sum(u^2) into a device scalar (one atomic per block)
//   scale   : X <- X / max(sqrt(sumsq), eps)          (Frobenius normalisation, in place)
//   update  : p <- p * (1 - lr*wd) - lr_adj * X       (bf16 direction, fp32 or bf16 parameter)
// All three are single passes with 16-byte accesses.
#include "common.cuh"

namespace {
using namespace fsb;

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

template <typename GT>
__global__ void __launch_bounds__(256)
muon_prepare_kernel(float* __restrict__ mom, const GT* __restrict__ g, __nv_bfloat16* __restrict__ u,
                    float* __restrict__ sumsq, long long n, float mu, int nesterov) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gv = static_cast<float>(g[i]);
    float m = mom[i];
    m = m + (1.f - mu) * (gv - m);
    mom[i] = m;
    const float uv = nesterov ? gv + mu * (m - gv) : m;
    const __nv_bfloat16 ub = __float2bfloat16(uv);
    u[i] = ub;
    const float ur = __bfloat162float(ub);
    acc += ur * ur;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, t);
  }
}

__global__ void muon_scale_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ sumsq,
                                  long long n, float eps) {
  const float inv = 1.f / fmaxf(sqrtf(*sumsq), eps);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * inv);
}

template <typename PT>
__global__ void muon_update_kernel(PT* __restrict__ p, const __nv_bfloat16* __restrict__ x, long long n,
                                   float decay, float step) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float pv = static_cast<float>(p[i]) * decay - step * __bfloat162float(x[i]);
    p[i] = static_cast<PT>(pv);
  }
}

inline int grid_for(long long n) {
  long long b = (n + 1023) / 1024;
  if (b < 1) b = 1;
  if (b > 148 * 16) b = 148 * 16;
  return static_cast<int>(b);
}
}  // namespace

// sumsq must be zero on entry (one float per matrix).
FSB_API int fsb_muon_prepare(float* mom, const void* g, int g_fp32, void* u, float* sumsq, long long n,
                             float mu, int nesterov, cudaStream_t stream) {
  if (n <= 0) return FSB_OK;
  if (g_fp32)
    muon_prepare_kernel<float><<<grid_for(n), 256, 0, stream>>>(mom, static_cast<const float*>(g),
        static_cast<__nv_bfloat16*>(u), sumsq, n, mu, nesterov);
  else
    muon_prepare_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(mom, static_cast<const __nv_bfloat16*>(g),
        static_cast<__nv_bfloat16*>(u), sumsq, n, mu, nesterov);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

FSB_API int fsb_muon_scale(void* x, const float* sumsq, long long n, float eps, cudaStream_t stream) {
  if (n <= 0) return FSB_OK;
  muon_scale_kernel<<<grid_for(n), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(x), sumsq, n, eps);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// p <- p * decay - step * x
FSB_API int fsb_muon_update(void* p, int p_fp32, const void* x, long long n, float decay, float step,
                            cudaStream_t stream) {
  if (n <= 0) return FSB_OK;
  if (p_fp32)
    muon_update_kernel<float><<<grid_for(n), 256, 0, stream>>>(static_cast<float*>(p),
        static_cast<const __nv_bfloat16*>(x), n, decay, step);
  else
    muon_update_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p),
        static_cast<const __nv_bfloat16*>(x), n, decay, step);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
