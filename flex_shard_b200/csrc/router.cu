// Mixture-of-experts router: activation (sigmoid or softmax over the experts), biased top-k
// selection, weight normalisation and the per-expert token histogram in one pass over the logits.
// One warp per token; lane l holds experts l, l+32, ... (up to 256 experts). The selection bias is
// added for choosing only; the weights come from the unbiased scores (auxiliary-loss-free
// balancing). Ties go to the lower expert index.
#include "common.cuh"

namespace {
using namespace fsb;

constexpr int MAX_PER_LANE = 8;   // 256 experts
constexpr int MAX_K = 16;

__global__ void __launch_bounds__(256)
route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, long long T, int E, int k,
                  int softmax, int normalize, float scale, long long* __restrict__ idx_out,
                  float* __restrict__ w_out, float* __restrict__ counts) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* row = logits + t * E;
  float s[MAX_PER_LANE], sel[MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (softmax) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      s[j] = e < E ? __expf(s[j] - mx) : 0.f;
      sum += s[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) s[j] *= inv;
  } else {
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) s[j] = 1.f / (1.f + __expf(-s[j]));
  }
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    sel[j] = e < E ? s[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float my_w = 0.f;      // lane c keeps the weight of choice c
  int my_e = 0;
  float wsum = 0.f;
  for (int c = 0; c < k; ++c) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > bv) {   // ascending e inside a lane, so ties keep the lower index
        bv = sel[j];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    // the owner lane hands out the unbiased score and retires the entry
    float sc = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      if (lane + 32 * j == be) {
        sc = s[j];
        sel[j] = -INFINITY;
      }
    }
    sc = __shfl_sync(0xffffffffu, sc, be & 31);
    wsum += sc;
    if (lane == c) {
      my_w = sc;
      my_e = be;
    }
  }
  if (lane < k) {
    const float w = normalize ? my_w / (wsum + 1e-20f) * scale : my_w * scale;
    idx_out[t * k + lane] = my_e;
    w_out[t * k + lane] = w;
    if (counts) atomicAdd(counts + my_e, 1.0f);
  }
}

}  // namespace

// logits [T, E] fp32 (E <= 256), bias [E] fp32 or null, k <= 16. idx_out [T, k] int64, w_out [T, k]
// fp32, counts [E] fp32 (incremented; may be null).
FSB_API int fsb_route_topk(const float* logits, const float* bias, long long T, int E, int k, int softmax,
                           int normalize, float scale, long long* idx_out, float* w_out, float* counts,
                           cudaStream_t stream) {
  if (T <= 0 || E <= 0 || E > 32 * MAX_PER_LANE || k <= 0 || k > MAX_K || k > E) return FSB_ERR_BAD_ARG;
  const int threads = 256;
  const long long blocks = (T * 32 + threads - 1) / threads;
  route_topk_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(logits, bias, T, E, k, softmax, normalize,
                                                                           scale, idx_out, w_out, counts);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
