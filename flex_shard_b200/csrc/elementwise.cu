// Bandwidth-bound kernels of the training step: RMSNorm, RoPE, SwiGLU, fused
// cross-entropy, AdamW over a flat bucket shard, dtype casts and the
// descriptor-driven segment gather/cast/zero used by bucket packing.
// All loads and stores are 16-byte vectors where alignment allows.
#include "common.cuh"

namespace {

using namespace fsb;

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

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) {
    t = warp_max(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// ------------------------------------------------------------------ RMSNorm
// One CTA per row; D % 8 == 0. Optional residual: s = x + res is written to
// `sum_out` and normalised (the pre-norm residual stream update in one pass).
constexpr int NORM_THREADS = 256;

// Block-wide sum with one barrier: every thread adds the warp partials itself. `red` holds two
// sets of partials used alternately, so consecutive calls need no second barrier.
__device__ __forceinline__ float block_sum_once(float v, float* red, int& ph) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[ph * 8 + w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) t += red[ph * 8 + i];
  ph ^= 1;
  return t;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 q = __bfloat1622float2(h[j]);
    f[2 * j] = q.x;
    f[2 * j + 1] = q.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return v;
}

// The row stays in registers between the two passes (D <= 8192: up to four 8-element groups per thread).
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd, int D, float eps) {
  __shared__ float red[16];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * D;
  const __nv_bfloat16* rr = res ? res + row * D : nullptr;
  uint4 cache[4];
  float ss = 0.f;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int i = threadIdx.x * 8 + g * NORM_THREADS * 8;
    if (i < D) {
      uint4 v = *reinterpret_cast<const uint4*>(xr + i);
      float f[8];
      unpack8(v, f);
      if (rr) {
        float q[8];
        unpack8(*reinterpret_cast<const uint4*>(rr + i), q);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += q[j];
        // round through bf16 so the normalised value matches the stored sum
        v = pack8(f);
        *reinterpret_cast<uint4*>(sum_out + row * D + i) = v;
        unpack8(v, f);
      }
      cache[g] = v;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  int ph = 0;
  ss = block_sum_once(ss, red, ph);
  const float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0) rstd[row] = r;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int i = threadIdx.x * 8 + g * NORM_THREADS * 8;
    if (i < D) {
      float f[8], q[8];
      unpack8(cache[g], f);
      unpack8(*reinterpret_cast<const uint4*>(w + i), q);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * r * q[j];
      *reinterpret_cast<uint4*>(y + row * D + i) = pack8(f);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); optional `dres` is added to dx
// (gradient arriving on the residual branch). dw partials: each CTA handles
// ROWS_PER_CTA rows and writes one fp32 partial row. A row's dy and x stay in registers between
// the reduction and the output pass; the weights are loaded once per CTA.
constexpr int NORM_BWD_ROWS = 32;

// G = number of 2048-column groups a thread touches (D <= 2048 G). The CTAs form a persistent grid that walks the
// rows with stride gridDim.x; the next row's dy / x / residual-gradient vectors are loaded before the current row
// is reduced, so a CTA always has two rows of loads in flight (without that the row loop is a chain of
// load -> barrier -> store latencies: 0.175 ms for 8192 x 4096, four times the traffic's time).
template <int G>
__global__ void __launch_bounds__(NORM_THREADS, G <= 2 ? 2 : 1)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, long long T, int D) {
  __shared__ float red[16];
  float dwacc[G][8];
  uint4 wv[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[g][j] = 0.f;
    const int i = threadIdx.x * 8 + g * NORM_THREADS * 8;
    wv[g] = i < D ? *reinterpret_cast<const uint4*>(w + i) : make_uint4(0, 0, 0, 0);
  }
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  uint4 av[G], bv[G], ev[G];
  float r = 0.f;
  auto load_row = [&](long long row, uint4 (&a)[G], uint4 (&b)[G], uint4 (&e)[G], float& rs) {
    rs = rstd[row];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int i = threadIdx.x * 8 + g * NORM_THREADS * 8;
      const bool in = i < D;
      a[g] = in ? *reinterpret_cast<const uint4*>(dy + row * D + i) : zero4;
      b[g] = in ? *reinterpret_cast<const uint4*>(x + row * D + i) : zero4;
      e[g] = (in && dres != nullptr) ? *reinterpret_cast<const uint4*>(dres + row * D + i) : zero4;
    }
  };
  long long row = blockIdx.x;
  if (row < T) load_row(row, av, bv, ev, r);
  int ph = 0;
  for (; row < T; row += gridDim.x) {
    const long long next = row + gridDim.x;
    uint4 an[G], bn[G], en[G];
    float rn = 0.f;
    if (next < T) load_row(next, an, bn, en, rn);
    float dot = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float a[8], b[8], c[8];
      unpack8(av[g], a);
      unpack8(bv[g], b);
      unpack8(wv[g], c);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += a[j] * c[j] * b[j];
    }
    dot = block_sum_once(dot, red, ph);
    const float coef = dot * r * r * r / D;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int i = threadIdx.x * 8 + g * NORM_THREADS * 8;
      if (i < D) {
        float a[8], b[8], c[8], e[8], o[8];
        unpack8(av[g], a);
        unpack8(bv[g], b);
        unpack8(wv[g], c);
        unpack8(ev[g], e);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = a[j] * c[j] * r - b[j] * coef + e[j];
          dwacc[g][j] += a[j] * b[j] * r;
        }
        *reinterpret_cast<uint4*>(dx + row * D + i) = pack8(o);
      }
    }
    if (next < T) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        av[g] = an[g];
        bv[g] = bn[g];
        ev[g] = en[g];
      }
      r = rn;
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int i = threadIdx.x * 8 + g * NORM_THREADS * 8;
    if (i < D) {
      float* p = dw_partial + static_cast<long long>(blockIdx.x) * D + i;
      *reinterpret_cast<float4*>(p) = make_float4(dwacc[g][0], dwacc[g][1], dwacc[g][2], dwacc[g][3]);
      *reinterpret_cast<float4*>(p + 4) =
          make_float4(dwacc[g][4], dwacc[g][5], dwacc[g][6], dwacc[g][7]);
    }
  }
}

// Column sums of partial[P, D] in a fixed order (deterministic), out bf16 or fp32, optional accumulate.
__global__ void colsum_kernel(const float* __restrict__ partial, void* __restrict__ out, int P, int D,
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

// ------------------------------------------------------------------ RoPE
// Interleaved-pair rotation (x[2i], x[2i+1]) * (cos_i + i sin_i), fp32 math, in
// place on a [T, H, hd] view with row stride `row_stride` elements. `inverse`
// rotates by the conjugate (the backward pass). table = [S, hd/2, 2] (cos, sin);
// position of row t is t % S.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ table,
                            long long T, int S, int H, int hd, long long row_stride, int inverse) {
  const int half = hd / 2;
  const long long total = T * H * (half / 4);  // 4 pairs (8 elements) per thread
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int p4 = idx % (half / 4);
    const long long th = idx / (half / 4);
    const int h = th % H;
    const long long t = th / H;
    const int pos = t % S;
    __nv_bfloat16* px = x + t * row_stride + static_cast<long long>(h) * hd + p4 * 8;
    float f[8];
    load8(px, f);
    const float4* tb = reinterpret_cast<const float4*>(table + (static_cast<long long>(pos) * half + p4 * 4) * 2);
    const float4 cs0 = tb[0], cs1 = tb[1];
    const float c[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
    float s[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float sj = inverse ? -s[j] : s[j];
      o[2 * j] = f[2 * j] * c[j] - f[2 * j + 1] * sj;
      o[2 * j + 1] = f[2 * j] * sj + f[2 * j + 1] * c[j];
    }
    store8(px, o);
  }
}

// ------------------------------------------------------------------ SwiGLU
// gu = [T, 2F] with gate in columns [0,F) and up in [F,2F); h = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                                  long long T, int F) {
  const long long total = T * (F / 8);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / (F / 8);
    const int c = (idx % (F / 8)) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * F + c, g);
    load8(gu + t * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(h + t * F + c, o);
  }
}
// dgu = [dgate, dup] from dh; written into a [T, 2F] buffer (may alias nothing).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const long long total = T * (F / 8);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / (F / 8);
    const int c = (idx % (F / 8)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * 2 * F + c, g);
    load8(gu + t * 2 * F + F + c, u);
    load8(dh + t * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    }
    store8(dgu + t * 2 * F + c, dg);
    store8(dgu + t * 2 * F + F + c, du);
  }
}

// ------------------------------------------------------------------ cross entropy (forward + backward in one pass)
// One CTA per row of logits [T, V] (bf16, V % 8 == 0). Writes loss[row] (fp32,
// 0 for ignored targets) and overwrites the row with
// dlogits = (softmax - onehot) * grad_scale.
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                     float* __restrict__ loss, int V, long long ld, float grad_scale,
                     long long ignore_index) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long tgt = target[row];
  float mx = -INFINITY;
  for (int i = threadIdx.x * 8; i < V; i += CE_THREADS * 8) {
    float f[8];
    load8(lr + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
  }
  mx = block_max<CE_THREADS>(mx, red);
  float se = 0.f;
  for (int i = threadIdx.x * 8; i < V; i += CE_THREADS * 8) {
    float f[8];
    load8(lr + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
  }
  se = block_sum<CE_THREADS>(se, red);
  const bool ignored = (tgt == ignore_index);
  if (threadIdx.x == 0) {
    loss[row] = ignored ? 0.f : (logf(se) + mx - __bfloat162float(lr[tgt]));
  }
  __syncthreads();
  const float inv = ignored ? 0.f : grad_scale / se;
  for (int i = threadIdx.x * 8; i < V; i += CE_THREADS * 8) {
    float f[8];
    load8(lr + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - mx) * inv;
      if (!ignored && i + j == tgt) p -= grad_scale;
      f[j] = p;
    }
    store8(lr + i, f);
  }
}

// The same result with one read and one write of the logits: the row is held on chip between the passes,
// its first `smem_vecs` 16-byte vectors in shared memory and the rest (up to CE_RV per thread) in registers.
// While the row streams in, every thread keeps a running maximum and a sum of exponentials relative to it
// (rescaled when the maximum grows), so the exponentials of the first pass hide under the loads; the block
// then combines the (max, sum) pairs, and the final pass turns the resident row into gradients while the
// stores drain. One CTA per SM (the row takes nearly all of its shared memory).
constexpr int CE_RV = 4;
constexpr int CE_SMEM_VECS = 14336;   // 224 KB of the row in shared memory
__global__ void __launch_bounds__(CE_THREADS, 1)
cross_entropy_resident_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                              float* __restrict__ loss, int V, long long ld, float grad_scale,
                              long long ignore_index, int smem_vecs) {
  extern __shared__ __align__(16) uint4 rowv[];
  __shared__ float red[32];
  const float L2E = 1.4426950408889634f;
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  uint4* g = reinterpret_cast<uint4*>(lr);
  const long long tgt = target[row];
  const bool ignored = (tgt == ignore_index);
  const int nvec = V / 8;
  const int tid = threadIdx.x;
  float tgt_logit = 0.f;
  if (tid == 0 && !ignored) tgt_logit = __bfloat162float(lr[tgt]);
  float m = -INFINITY, s = 0.f;
  auto take = [&](const uint4& v) {
    float f[8];
    unpack8(v, f);
    float vm = fmaxf(fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])), fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7])));
    if (vm > m) {
      s *= exp2f((m - vm) * L2E);
      m = vm;
    }
    const float mo = -m * L2E;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += exp2f(fmaf(f[j], L2E, mo));
  };
  uint4 rv[CE_RV];
#pragma unroll
  for (int k = 0; k < CE_RV; ++k) {
    const int idx = smem_vecs + tid + k * CE_THREADS;
    rv[k] = idx < nvec ? g[idx] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);   // -inf: adds nothing
  }
  int i = tid;
  for (; i + 3 * CE_THREADS < smem_vecs; i += 4 * CE_THREADS) {
    const uint4 a = g[i], b = g[i + CE_THREADS], c = g[i + 2 * CE_THREADS], d = g[i + 3 * CE_THREADS];
    rowv[i] = a; rowv[i + CE_THREADS] = b; rowv[i + 2 * CE_THREADS] = c; rowv[i + 3 * CE_THREADS] = d;
    take(a); take(b); take(c); take(d);
  }
  for (; i < smem_vecs; i += CE_THREADS) {
    const uint4 a = g[i];
    rowv[i] = a;
    take(a);
  }
#pragma unroll
  for (int k = 0; k < CE_RV; ++k)
    if (smem_vecs + tid + k * CE_THREADS < nvec) take(rv[k]);
  const float mx = block_max<CE_THREADS>(m, red);
  const float se = block_sum<CE_THREADS>(m == -INFINITY ? 0.f : s * exp2f((m - mx) * L2E), red);
  if (tid == 0) loss[row] = ignored ? 0.f : (logf(se) + mx - tgt_logit);
  const float inv = ignored ? 0.f : grad_scale / se;
  const float mo = -mx * L2E;
  const int tv = ignored ? -1 : static_cast<int>(tgt >> 3), tj = static_cast<int>(tgt & 7);
  auto grad = [&](const uint4& v, int idx) {
    float f[8];
    unpack8(v, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = exp2f(fmaf(f[j], L2E, mo)) * inv;
    if (idx == tv) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j == tj) f[j] -= grad_scale;
    }
    g[idx] = pack8(f);
  };
  for (i = tid; i < smem_vecs; i += CE_THREADS) grad(rowv[i], i);   // each thread reads back what it stored itself
#pragma unroll
  for (int k = 0; k < CE_RV; ++k) {
    const int idx = smem_vecs + tid + k * CE_THREADS;
    if (idx < nvec) grad(rv[k], idx);
  }
}

// ------------------------------------------------------------------ AdamW over a flat shard
// p: fp32 or bf16 master; g: fp32 or bf16; m, v: fp32. Optional `p_lowp`
// receives the updated parameter as bf16 (the all-gather send buffer when the
// master is fp32). Matches torch.optim.AdamW (decoupled decay, bias correction,
// eps added after the sqrt), maximize=False, amsgrad=False.
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2_sqrt, grad_scale;
};
__device__ __forceinline__ void ld8(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) { load8(p, f); }
__device__ __forceinline__ void st8(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) { store8(p, f); }

__device__ __forceinline__ void adamw_update(float& pv, float gv, float& mv, float& vv, const AdamArgs& a) {
  gv *= a.grad_scale;
  pv *= (1.f - a.lr * a.weight_decay);
  mv = mv + (1.f - a.beta1) * (gv - mv);  // lerp, as torch does
  vv = a.beta2 * vv + (1.f - a.beta2) * gv * gv;
  const float denom = sqrtf(vv) / a.bias2_sqrt + a.eps;
  pv -= (a.lr / a.bias1) * (mv / denom);
}

// 8 elements per thread per iteration with 16-byte accesses; `n8` full groups, then a scalar tail.
template <typename PT, typename GT>
__global__ void __launch_bounds__(256)
adamw_kernel(PT* __restrict__ p, const GT* __restrict__ g, float* __restrict__ m,
             float* __restrict__ v, __nv_bfloat16* __restrict__ p_lowp, long long n, int vec_ok,
             AdamArgs a) {
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n8 = vec_ok ? n / 8 : 0;
  for (long long i = tid; i < n8; i += stride) {
    float pf[8], gf[8], mf[8], vf[8];
    ld8(p + i * 8, pf);
    ld8(g + i * 8, gf);
    ld8(m + i * 8, mf);
    ld8(v + i * 8, vf);
#pragma unroll
    for (int j = 0; j < 8; ++j) adamw_update(pf[j], gf[j], mf[j], vf[j], a);
    st8(p + i * 8, pf);
    st8(m + i * 8, mf);
    st8(v + i * 8, vf);
    if (p_lowp) store8(p_lowp + i * 8, pf);
  }
  for (long long i = n8 * 8 + tid; i < n; i += stride) {
    float pv = static_cast<float>(p[i]), mv = m[i], vv = v[i];
    adamw_update(pv, static_cast<float>(g[i]), mv, vv, a);
    p[i] = static_cast<PT>(pv);
    m[i] = mv;
    v[i] = vv;
    if (p_lowp) p_lowp[i] = __float2bfloat16(pv);
  }
}

// ------------------------------------------------------------------ casts
template <typename ST, typename DT>
__global__ void cast_scale_kernel(const ST* __restrict__ s, DT* __restrict__ d, long long n, float scale,
                                  int accumulate) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f = static_cast<float>(s[i]) * scale;
    if (accumulate) f += static_cast<float>(d[i]);
    d[i] = static_cast<DT>(f);
  }
}

// fp32 [T, C] (row stride lds) -> bf16 [T, C] (row stride ldd); C % 4 == 0.
__global__ void cast2d_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d,
                                       long long T, int C, long long lds, long long ldd) {
  const long long total = T * (C / 4);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / (C / 4);
    const int c = (idx % (C / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(s + t * lds + c);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(d + t * ldd + c) = o;
  }
}

// ------------------------------------------------------------------ segment gather / cast / zero
// One descriptor per segment chunk. mode: 0 copy bytes, 1 fp32->bf16,
// 2 bf16->fp32, 3 zero-fill dst bytes. `n` counts bytes for modes 0/3 and
// elements for modes 1/2. Descriptors live in device memory.
struct SegDesc {
  const void* src;
  void* dst;
  long long n;
  int mode;
  int pad;
};
// 16-byte vectors, four in flight per thread: a long segment is a streaming copy and needs the loads of
// many iterations outstanding to fill the memory pipeline.
template <typename LoadStore>
__device__ __forceinline__ void seg_loop4(long long nv, long long tid, long long stride, LoadStore body) {
  long long i = tid;
  for (; i + 3 * stride < nv; i += 4 * stride) body(i, i + stride, i + 2 * stride, i + 3 * stride, 4);
  for (; i < nv; i += stride) body(i, i, i, i, 1);
}

__global__ void __launch_bounds__(256) segment_kernel(const SegDesc* __restrict__ descs, int chunks_per_seg) {
  const SegDesc d = descs[blockIdx.y];
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  (void)chunks_per_seg;
  const uintptr_t sa = reinterpret_cast<uintptr_t>(d.src), da = reinterpret_cast<uintptr_t>(d.dst);
  if (d.mode == 0 || d.mode == 3) {
    uint8_t* dst = static_cast<uint8_t*>(d.dst);
    const uint8_t* src = static_cast<const uint8_t*>(d.src);
    const bool zero = d.mode == 3;
    if (((da | (zero ? 0 : sa)) & 15) == 0) {
      const long long nv = d.n / 16;
      uint4* dv = reinterpret_cast<uint4*>(dst);
      const uint4* sv = reinterpret_cast<const uint4*>(src);
      if (zero) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (long long i = tid; i < nv; i += stride) dv[i] = z;
      } else {
        seg_loop4(nv, tid, stride, [&](long long i0, long long i1, long long i2, long long i3, int cnt) {
          if (cnt == 4) {
            const uint4 a = sv[i0], b = sv[i1], c = sv[i2], e = sv[i3];
            dv[i0] = a; dv[i1] = b; dv[i2] = c; dv[i3] = e;
          } else {
            dv[i0] = sv[i0];
          }
        });
      }
      for (long long i = nv * 16 + tid; i < d.n; i += stride) dst[i] = zero ? 0 : src[i];
    } else if (((da | (zero ? 0 : sa)) & 3) == 0 && (d.n & 3) == 0) {
      for (long long i = tid; i < d.n / 4; i += stride)
        reinterpret_cast<uint32_t*>(dst)[i] = zero ? 0u : reinterpret_cast<const uint32_t*>(src)[i];
    } else {
      for (long long i = tid; i < d.n; i += stride) dst[i] = zero ? 0 : src[i];
    }
  } else if (d.mode == 1) {
    const float* src = static_cast<const float*>(d.src);
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(d.dst);
    long long done = 0;
    if (((sa | da) & 15) == 0) {   // eight elements per vector: two float4 in, one 16-byte store out
      const long long nv = d.n / 8;
      const float4* sv = reinterpret_cast<const float4*>(src);
      uint4* dv = reinterpret_cast<uint4*>(dst);
      auto cvt = [](const float4& lo, const float4& hi) {
        uint4 o;
        o.x = pack_bf16x2(lo.x, lo.y); o.y = pack_bf16x2(lo.z, lo.w);
        o.z = pack_bf16x2(hi.x, hi.y); o.w = pack_bf16x2(hi.z, hi.w);
        return o;
      };
      seg_loop4(nv, tid, stride, [&](long long i0, long long i1, long long i2, long long i3, int cnt) {
        if (cnt == 4) {
          const float4 a0 = sv[2 * i0], a1 = sv[2 * i0 + 1], b0 = sv[2 * i1], b1 = sv[2 * i1 + 1];
          const float4 c0 = sv[2 * i2], c1 = sv[2 * i2 + 1], e0 = sv[2 * i3], e1 = sv[2 * i3 + 1];
          dv[i0] = cvt(a0, a1); dv[i1] = cvt(b0, b1); dv[i2] = cvt(c0, c1); dv[i3] = cvt(e0, e1);
        } else {
          dv[i0] = cvt(sv[2 * i0], sv[2 * i0 + 1]);
        }
      });
      done = nv * 8;
    }
    for (long long i = done + tid; i < d.n; i += stride) dst[i] = __float2bfloat16(src[i]);
  } else {
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(d.src);
    float* dst = static_cast<float*>(d.dst);
    long long done = 0;
    if (((sa | da) & 15) == 0) {   // eight elements per vector: one 16-byte load in, two float4 out
      const long long nv = d.n / 8;
      const uint4* sv = reinterpret_cast<const uint4*>(src);
      float4* dv = reinterpret_cast<float4*>(dst);
      auto put = [&](long long i, const uint4& v) {
        // a bf16 is the upper half of the fp32 with the same value
        dv[2 * i] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                                __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
        dv[2 * i + 1] = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                                    __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
      };
      seg_loop4(nv, tid, stride, [&](long long i0, long long i1, long long i2, long long i3, int cnt) {
        if (cnt == 4) {
          const uint4 a = sv[i0], b = sv[i1], c = sv[i2], e = sv[i3];
          put(i0, a); put(i1, b); put(i2, c); put(i3, e);
        } else {
          put(i0, sv[i0]);
        }
      });
      done = nv * 8;
    }
    for (long long i = done + tid; i < d.n; i += stride) dst[i] = __bfloat162float(src[i]);
  }
}

inline int grid_for(long long n, int threads, int per_thread = 1) {
  long long b = (n + static_cast<long long>(threads) * per_thread - 1) / (static_cast<long long>(threads) * per_thread);
  if (b < 1) b = 1;
  if (b > 148 * 16) b = 148 * 16;
  return static_cast<int>(b);
}
inline int launch_ok() { return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH; }

}  // namespace

FSB_API int fsb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out,
                            float* rstd, long long T, int D, float eps, cudaStream_t stream) {
  if (D % 8 != 0 || D > 8192 || T <= 0) return FSB_ERR_BAD_ARG;
  rmsnorm_fwd_kernel<<<static_cast<unsigned>(T), NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
      static_cast<__nv_bfloat16*>(sum_out), rstd, D, eps);
  return launch_ok();
}

// dw_partial must hold ceil(T/32) * D floats. dw_out: bf16 or fp32 [D].
FSB_API int fsb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                            const void* dres, void* dx, float* dw_partial, void* dw_out,
                            int dw_fp32, int dw_accumulate, long long T, int D,
                            cudaStream_t stream) {
  if (D % 8 != 0 || D > 8192 || T <= 0) return FSB_ERR_BAD_ARG;
  // dw_partial holds ceil(T / 32) rows (the caller's contract); the persistent grid uses at most that many CTAs
  // and at most two per SM
  int blocks = static_cast<int>((T + NORM_BWD_ROWS - 1) / NORM_BWD_ROWS);
  static int sms = 0;
  if (sms == 0 && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0) != cudaSuccess) sms = 148;
  const int groups = (D + NORM_THREADS * 8 - 1) / (NORM_THREADS * 8);
  const int per_sm = groups <= 2 ? 2 : 1;     // wide rows keep three double-buffered vectors per group in registers
  if (blocks > per_sm * sms) blocks = per_sm * sms;
  auto launch = [&](auto kernel) {
    kernel<<<blocks, NORM_THREADS, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
        static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),
        static_cast<__nv_bfloat16*>(dx), dw_partial, T, D);
  };
  if (groups == 1) launch(rmsnorm_bwd_kernel<1>);
  else if (groups == 2) launch(rmsnorm_bwd_kernel<2>);
  else if (groups == 3) launch(rmsnorm_bwd_kernel<3>);
  else launch(rmsnorm_bwd_kernel<4>);
  colsum_kernel<<<(D + 255) / 256, 256, 0, stream>>>(dw_partial, dw_out, blocks, D, dw_fp32,
                                                      dw_accumulate);
  return launch_ok();
}

FSB_API int fsb_rope(void* x, const float* table, long long T, int S, int H, int hd,
                     long long row_stride, int inverse, cudaStream_t stream) {
  if (hd % 16 != 0 || row_stride % 8 != 0) return FSB_ERR_BAD_ARG;
  const long long total = T * H * (hd / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(x), table, T, S,
                                                        H, hd, row_stride, inverse);
  return launch_ok();
}

FSB_API int fsb_swiglu_fwd(const void* gu, void* h, long long T, int F, cudaStream_t stream) {
  if (F % 8 != 0) return FSB_ERR_BAD_ARG;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), T, F);
  return launch_ok();
}
FSB_API int fsb_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long T, int F,
                           cudaStream_t stream) {
  if (F % 8 != 0) return FSB_ERR_BAD_ARG;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh),
      static_cast<__nv_bfloat16*>(dgu), T, F);
  return launch_ok();
}

FSB_API int fsb_cross_entropy(void* logits, const long long* target, float* loss, long long T, int V,
                              long long ld, float grad_scale, long long ignore_index,
                              cudaStream_t stream) {
  if (V % 8 != 0 || ld % 8 != 0) return FSB_ERR_BAD_ARG;
  const int nvec = V / 8;
  const int smem_vecs = nvec < CE_SMEM_VECS ? nvec : CE_SMEM_VECS;
  if ((reinterpret_cast<uintptr_t>(logits) & 15) == 0 && nvec - smem_vecs <= CE_RV * CE_THREADS) {
    // the row fits on chip: one read and one write
    const size_t smem = static_cast<size_t>(smem_vecs) * 16;
    if (cudaFuncSetAttribute(cross_entropy_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FSB_ERR_LAUNCH;
    cross_entropy_resident_kernel<<<static_cast<unsigned>(T), CE_THREADS, smem, stream>>>(
        static_cast<__nv_bfloat16*>(logits), target, loss, V, ld, grad_scale, ignore_index, smem_vecs);
    return launch_ok();
  }
  cross_entropy_kernel<<<static_cast<unsigned>(T), CE_THREADS, 0, stream>>>(
      static_cast<__nv_bfloat16*>(logits), target, loss, V, ld, grad_scale, ignore_index);
  return launch_ok();
}

// The same with the descriptor table left in page-locked host memory: every CTA fetches its own 32-byte
// record over the host link, which saves the table's host-to-device copy (a copy-engine operation between
// two kernels of the same stream costs more than the fetch for the few dozen records of a bucket).
// Returns FSB_ERR_BAD_ARG when the table is not device-accessible page-locked memory.
FSB_API int fsb_segment_op_host(const void* host_descs, int nseg, int blocks_per_seg, cudaStream_t stream) {
  if (nseg <= 0) return FSB_OK;
  if (nseg > 65535) return FSB_ERR_TOO_LARGE;
  void* dptr = nullptr;
  if (cudaHostGetDevicePointer(&dptr, const_cast<void*>(host_descs), 0) != cudaSuccess || dptr == nullptr) {
    (void)cudaGetLastError();
    return FSB_ERR_BAD_ARG;
  }
  if (blocks_per_seg < 1) blocks_per_seg = 1;
  dim3 grid(blocks_per_seg, nseg);
  segment_kernel<<<grid, 256, 0, stream>>>(static_cast<const SegDesc*>(dptr), blocks_per_seg);
  return launch_ok();
}

// step >= 1. p_fp32 / g_fp32 select the master and gradient dtypes.
FSB_API int fsb_adamw(void* p, const void* g, float* m, float* v, void* p_lowp, long long n,
                      int p_fp32, int g_fp32, float lr, float beta1, float beta2, float eps,
                      float weight_decay, int step, float grad_scale, cudaStream_t stream) {
  if (n <= 0) return FSB_OK;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bias2_sqrt = sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  a.grad_scale = grad_scale;
  const int grid = grid_for(n, 256, 8);
  __nv_bfloat16* lp = static_cast<__nv_bfloat16*>(p_lowp);
  const uintptr_t al = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                       reinterpret_cast<uintptr_t>(p_lowp);
  const int vec = (al & 15) == 0;
  if (p_fp32 && g_fp32)
    adamw_kernel<float, float><<<grid, 256, 0, stream>>>(static_cast<float*>(p), static_cast<const float*>(g), m, v, lp, n, vec, a);
  else if (p_fp32)
    adamw_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<float*>(p), static_cast<const __nv_bfloat16*>(g), m, v, lp, n, vec, a);
  else if (g_fp32)
    adamw_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p), static_cast<const float*>(g), m, v, lp, n, vec, a);
  else
    adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(g), m, v, lp, n, vec, a);
  return launch_ok();
}

// mode: 1 fp32->bf16, 2 bf16->fp32, 4 fp32->fp32, 5 bf16->bf16 (scale / accumulate variants).
FSB_API int fsb_cast_scale(const void* src, void* dst, long long n, int mode, float scale,
                           int accumulate, cudaStream_t stream) {
  if (n <= 0) return FSB_OK;
  const int grid = grid_for(n, 256, 4);
  switch (mode) {
    case 1: cast_scale_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n, scale, accumulate); break;
    case 2: cast_scale_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n, scale, accumulate); break;
    case 4: cast_scale_kernel<float, float><<<grid, 256, 0, stream>>>(static_cast<const float*>(src), static_cast<float*>(dst), n, scale, accumulate); break;
    case 5: cast_scale_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), n, scale, accumulate); break;
    default: return FSB_ERR_BAD_ARG;
  }
  return launch_ok();
}

FSB_API int fsb_cast2d_f32_bf16(const float* src, void* dst, long long T, int C, long long lds,
                                long long ldd, cudaStream_t stream) {
  if (C % 4 != 0 || lds % 4 != 0 || ldd % 4 != 0) return FSB_ERR_BAD_ARG;
  cast2d_f32_bf16_kernel<<<grid_for(T * (C / 4), 256), 256, 0, stream>>>(
      src, static_cast<__nv_bfloat16*>(dst), T, C, lds, ldd);
  return launch_ok();
}

// descs: device array of `nseg` SegDesc records (32 bytes: src, dst, n, mode, pad).
FSB_API int fsb_segment_op(const void* descs, int nseg, int blocks_per_seg, cudaStream_t stream) {
  if (nseg <= 0) return FSB_OK;
  if (nseg > 65535) return FSB_ERR_TOO_LARGE;
  if (blocks_per_seg < 1) blocks_per_seg = 1;
  dim3 grid(blocks_per_seg, nseg);
  segment_kernel<<<grid, 256, 0, stream>>>(static_cast<const SegDesc*>(descs), blocks_per_seg);
  return launch_ok();
}
