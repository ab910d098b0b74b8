// Muon's elementwise passes around the Newton-Schulz GEMMs (which run on gemm_bf16.cu):
//   prepare : M <- lerp(M, g, 1-mu); u = nesterov ? lerp(g, M, mu) : M; write u as bf16 and
//             sum(u^2): every block writes its partial sum to a workspace slot and the block that
//             finishes last adds the slots in index order, so the result does not depend on the
//             order in which blocks ran
//   scale   : X <- X / max(sqrt(sumsq), eps)          (Frobenius normalisation, in place)
//   update  : p <- p * (1 - lr*wd) - lr_adj * X       (bf16 direction, fp32 or bf16 parameter)
// Eight elements per thread and iteration (16-byte accesses) when the pointers are 16-byte aligned;
// a scalar loop covers the tail and unaligned tensors.
#include "common.cuh"

namespace {
using namespace fsb;

constexpr int kMaxBlocks = 148 * 16;
// workspace layout (floats): [0] sum of squares, [1] finished-block counter (as uint), [2 .. 2+kMaxBlocks) partials
constexpr int kWsFloats = 2 + kMaxBlocks;

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xffff0000u);
  v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xffff0000u);
  v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xffff0000u);
  v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xffff0000u);
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float block_sum_256(float acc, float* red) {
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) t = warp_sum(t);
  return t;   // valid in thread 0
}

template <typename GT>
__global__ void __launch_bounds__(256)
muon_prepare_kernel(float* __restrict__ mom, const GT* __restrict__ g, __nv_bfloat16* __restrict__ u,
                    float* __restrict__ ws, long long n, float mu, int nesterov) {
  __shared__ float red[8];
  __shared__ int last;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float acc = 0.f;
  auto one = [&](float gv, float m, float& m_out) {
    m = m + (1.f - mu) * (gv - m);
    m_out = m;
    return nesterov ? gv + mu * (m - gv) : m;
  };
  long long done = 0;
  if (aligned16(mom) && aligned16(g) && aligned16(u)) {
    const long long nv = n / 8;
    for (long long i = tid; i < nv; i += stride) {
      float gv[8], m[8], uv[8];
      load8(g + i * 8, gv);
      load8(mom + i * 8, m);
#pragma unroll
      for (int j = 0; j < 8; ++j) uv[j] = one(gv[j], m[j], m[j]);
      store8(mom + i * 8, m);
      store8(u + i * 8, uv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float ur = __bfloat162float(__float2bfloat16(uv[j]));   // the norm is that of the rounded matrix
        acc += ur * ur;
      }
    }
    done = nv * 8;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float m;
    const float uv = one(static_cast<float>(g[i]), mom[i], m);
    mom[i] = m;
    const __nv_bfloat16 ub = __float2bfloat16(uv);
    u[i] = ub;
    const float ur = __bfloat162float(ub);
    acc += ur * ur;
  }
  const float t = block_sum_256(acc, red);
  if (threadIdx.x == 0) {
    ws[2 + blockIdx.x] = t;
    __threadfence();
    const unsigned prev = atomicAdd(reinterpret_cast<unsigned*>(ws + 1), 1u);
    last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // the last block to finish: add the partials in index order (a fixed order whatever the schedule was)
  float s = 0.f;
  for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += 256) s += __ldcg(ws + 2 + i);
  __syncthreads();
  const float total = block_sum_256(s, red);
  if (threadIdx.x == 0) {
    ws[0] = total;
    *reinterpret_cast<unsigned*>(ws + 1) = 0u;   // ready for the next use of the workspace
  }
}

__global__ void __launch_bounds__(256)
muon_scale_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ sumsq, long long n, float eps) {
  const float inv = 1.f / fmaxf(sqrtf(*sumsq), eps);
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long done = 0;
  if (aligned16(x)) {
    const long long nv = n / 8;
    for (long long i = tid; i < nv; i += stride) {
      float v[8];
      load8(x + i * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= inv;
      store8(x + i * 8, v);
    }
    done = nv * 8;
  }
  for (long long i = done + tid; i < n; i += stride) x[i] = __float2bfloat16(__bfloat162float(x[i]) * inv);
}

template <typename PT>
__global__ void __launch_bounds__(256)
muon_update_kernel(PT* __restrict__ p, const __nv_bfloat16* __restrict__ x, long long n, float decay, float step) {
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long done = 0;
  if (aligned16(p) && aligned16(x)) {
    const long long nv = n / 8;
    for (long long i = tid; i < nv; i += stride) {
      float pv[8], xv[8];
      load8(p + i * 8, pv);
      load8(x + i * 8, xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) pv[j] = pv[j] * decay - step * xv[j];
      store8(p + i * 8, pv);
    }
    done = nv * 8;
  }
  for (long long i = done + tid; i < n; i += stride)
    p[i] = static_cast<PT>(static_cast<float>(p[i]) * decay - step * __bfloat162float(x[i]));
}

inline int grid_for(long long n) {
  long long b = (n + 2047) / 2048;   // 256 threads x 8 elements
  if (b < 1) b = 1;
  if (b > kMaxBlocks) b = kMaxBlocks;
  return static_cast<int>(b);
}
}  // namespace

// Floats a workspace needs (it must be zero before its first use; a finished call leaves it reusable).
FSB_API int fsb_muon_workspace_floats() { return kWsFloats; }

// ws: workspace of fsb_muon_workspace_floats() floats; ws[0] receives sum(u^2).
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
