// Row movement for mixture-of-experts layers: token rows are gathered into an expert-major,
// 128-row-aligned layout for the grouped tcgen05 GEMMs and combined back with the routing weights.
// One warp per row, 16-byte accesses; indices and weights stay on the device (no host sync).
#include "common.cuh"

namespace {
using namespace fsb;

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

// dst[i, :] = scale[i] * src[index[i], :]   (index < 0 -> zero row; scale may be null)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ index,
                                   const float* __restrict__ scale, __nv_bfloat16* __restrict__ dst,
                                   long long n, int D, long long lds, long long ldd) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= n) return;
  const int s = index[w];
  const float sc = (scale != nullptr && s >= 0) ? scale[w] : 1.f;
  for (int c = lane * 8; c < D; c += 256) {
    bf16x8 v;
    if (s >= 0) {
      v = *reinterpret_cast<const bf16x8*>(src + static_cast<long long>(s) * lds + c);
      if (scale != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(v.v[j]);
          v.v[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v.v[j] = __floats2bfloat162_rn(0.f, 0.f);
    }
    *reinterpret_cast<bf16x8*>(dst + w * ldd + c) = v;
  }
}

// out[t, :] = sum_k w[t, k] * rows[pos[t, k], :]   (w may be null: plain sum)
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ pos,
                                    const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                    long long T, int k, int D, long long ldr, long long ldo) {
  const long long t = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane * 8; c < D; c += 256) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int p = pos[t * k + j];
      if (p < 0) continue;
      const float wj = w ? w[t * k + j] : 1.f;
      const bf16x8 v = *reinterpret_cast<const bf16x8*>(rows + static_cast<long long>(p) * ldr + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(v.v[q]);
        acc[2 * q] += wj * f.x;
        acc[2 * q + 1] += wj * f.y;
      }
    }
    bf16x8 o;
#pragma unroll
    for (int q = 0; q < 4; ++q) o.v[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<bf16x8*>(out + t * ldo + c) = o;
  }
}

// dw[t, k] = <dy[t, :], rows[pos[t, k], :]>
__global__ void combine_bwd_w_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ rows,
                                     const int* __restrict__ pos, float* __restrict__ dw, long long TK, int k,
                                     int D, long long lddy, long long ldr) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= TK) return;
  const long long t = i / k;
  const int p = pos[i];
  float acc = 0.f;
  if (p >= 0) {
    for (int c = lane * 8; c < D; c += 256) {
      const bf16x8 a = *reinterpret_cast<const bf16x8*>(dy + t * lddy + c);
      const bf16x8 b = *reinterpret_cast<const bf16x8*>(rows + static_cast<long long>(p) * ldr + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __bfloat1622float2(a.v[q]), y = __bfloat1622float2(b.v[q]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dw[i] = acc;
}

inline unsigned blocks_for_warps(long long warps) {
  return static_cast<unsigned>((warps * 32 + 255) / 256);
}
inline int ok() { return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH; }
}  // namespace

FSB_API int fsb_moe_gather_rows(const void* src, const int* index, const float* scale, void* dst, long long n,
                                int D, long long lds, long long ldd, cudaStream_t stream) {
  if (D % 8 != 0 || lds % 8 != 0 || ldd % 8 != 0) return FSB_ERR_BAD_ARG;
  if (n <= 0) return FSB_OK;
  gather_rows_kernel<<<blocks_for_warps(n), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), index, scale,
                                                             static_cast<__nv_bfloat16*>(dst), n, D, lds, ldd);
  return ok();
}

FSB_API int fsb_moe_combine_rows(const void* rows, const int* pos, const float* w, void* out, long long T, int k,
                                 int D, long long ldr, long long ldo, cudaStream_t stream) {
  if (D % 8 != 0 || ldr % 8 != 0 || ldo % 8 != 0) return FSB_ERR_BAD_ARG;
  if (T <= 0) return FSB_OK;
  combine_rows_kernel<<<blocks_for_warps(T), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(rows), pos, w,
                                                              static_cast<__nv_bfloat16*>(out), T, k, D, ldr, ldo);
  return ok();
}

FSB_API int fsb_moe_combine_bwd_w(const void* dy, const void* rows, const int* pos, float* dw, long long T, int k,
                                  int D, long long lddy, long long ldr, cudaStream_t stream) {
  if (D % 8 != 0) return FSB_ERR_BAD_ARG;
  if (T <= 0) return FSB_OK;
  combine_bwd_w_kernel<<<blocks_for_warps(T * k), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(rows), pos, dw, T * k, k, D, lddy, ldr);
  return ok();
}

// ------------------------------------------------------------------ route planning in one launch
// Stable expert-major ordering of n = T*k (token, choice) pairs with every expert's block padded to 128
// rows: histogram, padded prefix sums, tile -> expert table and the row of every pair, all by ONE CTA.
// Each of the 32 warps owns a contiguous chunk of pairs; within a 32-pair step the lanes that chose the
// same expert find each other with match.any, which gives every pair its stable rank without atomics.
namespace {
constexpr int kPlanWarps = 32;
constexpr int kPlanMaxExperts = 256;

__global__ void __launch_bounds__(kPlanWarps * 32)
plan_routes_kernel(const long long* __restrict__ idx64, const int* __restrict__ idx32, long long n, int k, int E,
                   long long max_rows, int* __restrict__ pos, int* __restrict__ src, int* __restrict__ offs,
                   int* __restrict__ tile_expert, int* __restrict__ num_mtiles, int* __restrict__ counts) {
  extern __shared__ int sm[];
  int* cnt = sm;                              // [warps][E] counts, then running offsets
  int* off = sm + kPlanWarps * E;             // [E + 1] padded offsets
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long chunk = (n + kPlanWarps - 1) / kPlanWarps;
  const long long lo = warp * chunk, hi = lo + chunk < n ? lo + chunk : n;
  for (int i = threadIdx.x; i < kPlanWarps * E; i += blockDim.x) cnt[i] = 0;
  for (long long i = threadIdx.x; i < max_rows; i += blockDim.x) src[i] = -1;
  __syncthreads();
  auto expert_of = [&](long long i) { return idx64 ? static_cast<int>(idx64[i]) : idx32[i]; };
  // phase 1: per-warp histogram
  for (long long base = lo; base < hi; base += 32) {
    const long long i = base + lane;
    const bool live = i < hi;
    const unsigned act = __ballot_sync(0xffffffffu, live);
    if (live) {
      const int e = expert_of(i);
      const unsigned same = __match_any_sync(act, e);
      if ((same & ((1u << lane) - 1)) == 0) cnt[warp * E + e] += __popc(same);
    }
    __syncwarp();
  }
  __syncthreads();
  // phase 2: totals, exclusive scan over warps, padded offsets
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < kPlanWarps; ++w) {
      const int c = cnt[w * E + e];
      cnt[w * E + e] = run;
      run += c;
    }
    if (counts != nullptr) counts[e] = run;
    off[e + 1] = (run + 127) / 128 * 128;     // padded size of expert e, turned into an offset below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    off[0] = 0;
    for (int e = 0; e < E; ++e) off[e + 1] += off[e];
    *num_mtiles = off[E] / 128;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offs[e] = off[e];
  for (long long t = threadIdx.x; t < max_rows / 128; t += blockDim.x) {
    // expert of m-tile t: the first expert whose padded block ends after the tile's first row (empty experts
    // end where they start and are skipped); tiles past the last block map to the last expert
    const int row = static_cast<int>(t) * 128;
    int a = 0, b = E;                         // first e in [0, E) with off[e + 1] > row, else E
    while (a < b) {
      const int mid = (a + b) / 2;
      if (off[mid + 1] > row) b = mid; else a = mid + 1;
    }
    tile_expert[t] = a < E ? a : E - 1;
  }
  // phase 3: rows
  for (long long base = lo; base < hi; base += 32) {
    const long long i = base + lane;
    const bool live = i < hi;
    const unsigned act = __ballot_sync(0xffffffffu, live);
    if (live) {
      const int e = expert_of(i);
      const unsigned same = __match_any_sync(act, e);
      const int rank_in_step = __popc(same & ((1u << lane) - 1));
      const int row = off[e] + cnt[warp * E + e] + rank_in_step;
      pos[i] = row;
      src[row] = static_cast<int>(i / k);
      __syncwarp(act);
      if (rank_in_step == 0) cnt[warp * E + e] += __popc(same);
    }
    __syncwarp();
  }
}
}  // namespace

// idx: n expert ids (int64 when idx_is_i64 else int32). Outputs are int32 device arrays: pos[n], src[max_rows],
// offs[E + 1], tile_expert[max_rows / 128], num_mtiles[1], counts[E] (pairs per expert; may be null). max_rows
// must be a multiple of 128 that covers the padded layout in the worst case.
FSB_API int fsb_moe_plan_routes(const void* idx, int idx_is_i64, long long n, int k, int E, long long max_rows,
                                int* pos, int* src, int* offs, int* tile_expert, int* num_mtiles, int* counts,
                                cudaStream_t stream) {
  if (E <= 0 || E > kPlanMaxExperts || k <= 0 || n < 0 || max_rows % 128 != 0) return FSB_ERR_BAD_ARG;
  const size_t smem = (static_cast<size_t>(kPlanWarps) * E + E + 1) * sizeof(int);
  plan_routes_kernel<<<1, kPlanWarps * 32, smem, stream>>>(
      idx_is_i64 ? static_cast<const long long*>(idx) : nullptr, idx_is_i64 ? nullptr : static_cast<const int*>(idx),
      n, k, E, max_rows, pos, src, offs, tile_expert, num_mtiles, counts);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
