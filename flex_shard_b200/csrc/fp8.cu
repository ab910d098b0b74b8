// Blockwise FP8 (e4m3) support for sm_100a:
//   * weight quantiser: one fp32 scale per 128x128 tile (amax/448), stored as its reciprocal
//     ("dequant scale"), a pure function of the tile so that quantising a rank's rows locally
//     equals quantising after a bf16 gather bit for bit;
//   * activation quantiser: one scale per (row, 128-column group), written k-block major;
//   * block-scaled GEMM: tcgen05.mma kind::f8f6f4 accumulates one 128-deep K block at a time in
//     TMEM; the epilogue warps fold each block into fp32 registers with its (row, k-block) x
//     (n-block, k-block) scale while the tensor core already works on the next block.
//
//   D[M,N] (bf16) = sum_kb sa[kb][m] * sb(n/128, kb) * (Aq[m, kb] . Bq[n, kb]^T)
//
// A is K-major e4m3 [M, K]. B is e4m3, either K-major [N, K] (forward: B = W) or MN-major
// [K, N] (dgrad: B = W read as its transpose), with the weight's 128x128 scales indexed through
// two strides.
#include "common.cuh"
#include <cuda_fp8.h>

namespace {
using namespace fsb;

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

// ------------------------------------------------------------------ weight quantiser (128x128 tiles)
// grid = (ceil(cols/128), ceil(rows/128)); 256 threads; each thread owns 8 columns x 8 rows.
__global__ void __launch_bounds__(256)
quant_weight_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                            float* __restrict__ inv_scale, int rows, int cols, long long ldw,
                            long long ldq, int scale_cols) {
  __shared__ float red[8];
  const int tr = blockIdx.y * 128, tc = blockIdx.x * 128;
  const int cg = threadIdx.x & 15;   // 16 column groups of 8
  const int rg = threadIdx.x >> 4;   // 16 row groups of 8
  const int c0 = tc + cg * 8;
  float vals[8][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = tr + rg * 8 + i;
    if (r < rows && c0 + 8 <= cols) {
      const bf16x8 t = *reinterpret_cast<const bf16x8*>(w + r * ldw + c0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(t.v[j]);
        vals[i][2 * j] = f.x;
        vals[i][2 * j + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        vals[i][j] = (r < rows && c0 + j < cols) ? __bfloat162float(w[r * ldw + c0 + j]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vals[i][j]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  amax = fmaxf(amax, 1e-12f);
  const float scale = 448.f / amax;
  if (threadIdx.x == 0) inv_scale[blockIdx.y * scale_cols + blockIdx.x] = 1.f / scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = tr + rg * 8 + i;
    if (r >= rows) continue;
    uint8_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = fminf(fmaxf(vals[i][j] * scale, -448.f), 448.f);
      o[j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3));
    }
    if (c0 + 8 <= cols) {
      *reinterpret_cast<uint2*>(q + r * ldq + c0) = *reinterpret_cast<const uint2*>(o);
    } else {
      for (int j = 0; j < 8 && c0 + j < cols; ++j) q[r * ldq + c0 + j] = o[j];
    }
  }
}

// ------------------------------------------------------------------ activation quantiser (1x128 groups)
// One warp per (row, 128-column group); inv_scale is written [K/128, T] (k-block major).
__global__ void quant_act_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ inv_scale, long long T, int K, long long ldx,
                                       long long ldq) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = K / 128;
  if (w >= T * groups) return;
  const long long row = w / groups;
  const int g = w % groups;
  const __nv_bfloat16* p = x + row * ldx + g * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(b2[0]), b = __bfloat1622float2(b2[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = fmaxf(warp_max(amax), 1e-12f);
  const float scale = 448.f / amax;
  if (lane == 0) inv_scale[static_cast<long long>(g) * T + row] = 1.f / scale;
  uint8_t o[4];
  o[0] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(a.x * scale, __NV_SATFINITE, __NV_E4M3));
  o[1] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(a.y * scale, __NV_SATFINITE, __NV_E4M3));
  o[2] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(b.x * scale, __NV_SATFINITE, __NV_E4M3));
  o[3] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(b.y * scale, __NV_SATFINITE, __NV_E4M3));
  *reinterpret_cast<uint32_t*>(q + row * ldq + g * 128 + lane * 4) = *reinterpret_cast<const uint32_t*>(o);
}

// ------------------------------------------------------------------ block-scaled GEMM
constexpr int BM = 128, BN = 128, BK = 128;  // BK bytes == elements (fp8)
constexpr int STAGES = 5;
constexpr int A_STAGE = BM * BK, B_STAGE = BN * BK, STAGE_BYTES = A_STAGE + B_STAGE;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int NUM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 scale-accumulate (two per lane quarter)

struct Fp8Args {
  int M, N, K;
  int b_mn;
  const float* sa;            // [K/128][M]
  const float* sb;            // weight scales, addressed sb[nb * sb_stride_n + kb * sb_stride_k]
  long long sb_stride_n, sb_stride_k;
  __nv_bfloat16* d;
  long long ldd;
  int* status;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Fp8Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;       // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (args.M + BM - 1) / BM, tiles_n = (args.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = args.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(sa, &map_a, &full_bar[s], kb * BK, tm * BM);
          if (!args.b_mn) tma_load_2d(sb, &map_b, &full_bar[s], kb * BK, tn * BN);
          else tma_load_2d(sb, &map_b, &full_bar[s], tn * BN, kb * BK);  // [K rows][128 N bytes]
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop (waits and descriptor arithmetic stay warp-uniform); one elected
    // lane issues the tcgen05 instructions.
    {
      // e4m3 x e4m3 -> fp32; B MN-major for the transposed-weight product
      const uint32_t idesc = make_idesc(BM, BN, 0, 0, 0, args.b_mn ? 1u : 0u);
      // K-major: 32 elements (bytes) per MMA inside the 128-byte row. MN-major B: one 128-wide
      // N group, 8-deep K groups 1 KB apart, 32 K = 4 groups = 4 KB per MMA.
      const uint32_t b_kstep = (args.b_mn ? 4096u : 32u) >> 4;
      uint32_t it = 0, blk = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it, ++blk) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const uint32_t buf = blk & 1, bph = (blk >> 1) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag) || !mbar_wait(&tmem_empty[buf], bph ^ 1, abort_flag)) {
            if (lane == 0) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sa + A_STAGE, 16, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 32; ++k)
              umma_f8(tmem_base + buf * BN, da + k * 2, db + k * b_kstep, idesc, k != 0);
            umma_commit(&empty_bar[s]);
            umma_commit(&tmem_full[buf]);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // Two warps per TMEM lane quarter, each folding 64 of the tile's 128 columns.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HC = BN / 2;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t blk = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const long long row = static_cast<long long>(tm) * BM + quarter * 32 + lane;
      const bool row_ok = row < args.M;
      float acc[HC];
#pragma unroll
      for (int i = 0; i < HC; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++blk) {
        const uint32_t buf = blk & 1, bph = (blk >> 1) & 1;
        const float s = (row_ok ? args.sa[static_cast<long long>(kb) * args.M + row] : 0.f) *
                        args.sb[tn * args.sb_stride_n + kb * args.sb_stride_k];
        if (!mbar_wait(&tmem_full[buf], bph, abort_flag)) {
          if (lane == 0) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(tmem_base + lane_off + buf * BN + half * HC, v0);
        tmem_ld_32x32(tmem_base + lane_off + buf * BN + half * HC + 32, v1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);  // values are in registers: free the buffer early
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = fmaf(s, __uint_as_float(v0[i]), acc[i]);
          acc[32 + i] = fmaf(s, __uint_as_float(v1[i]), acc[32 + i]);
        }
      }
      if (ok && row_ok) {
        const int cbase = tn * BN + half * HC;
        __nv_bfloat16* dp = args.d + row * args.ldd + cbase;
        const int ncols = min(HC, args.N - cbase);
        if (ncols == HC && (args.ldd % 8) == 0) {
#pragma unroll
          for (int i = 0; i < HC; i += 8) {
            uint4 o;
            o.x = pack_bf16x2(acc[i], acc[i + 1]);
            o.y = pack_bf16x2(acc[i + 2], acc[i + 3]);
            o.z = pack_bf16x2(acc[i + 4], acc[i + 5]);
            o.w = pack_bf16x2(acc[i + 6], acc[i + 7]);
            *reinterpret_cast<uint4*>(dp + i) = o;
          }
        } else {
#pragma unroll
          for (int i = 0; i < HC; ++i)
            if (i < ncols) dp[i] = __float2bfloat16(acc[i]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      const unsigned long long t0 = clock64();
      while (clock64() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

int g_sms[64] = {0};
}  // namespace

// w: bf16 [rows, cols] (row stride ldw); q: e4m3 bytes [rows, cols] (row stride ldq);
// inv_scale: fp32 [ceil(rows/128), ceil(cols/128)].
FSB_API int fsb_fp8_quant_weight(const void* w, void* q, float* inv_scale, int rows, int cols, long long ldw,
                                 long long ldq, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return FSB_OK;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  quant_weight_128x128_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w),
                                                        static_cast<uint8_t*>(q), inv_scale, rows, cols, ldw,
                                                        ldq, (cols + 127) / 128);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// x: bf16 [T, K] with K % 128 == 0; q: e4m3 [T, K]; inv_scale: fp32 [K/128, T].
FSB_API int fsb_fp8_quant_act(const void* x, void* q, float* inv_scale, long long T, int K, long long ldx,
                              long long ldq, cudaStream_t stream) {
  if (K % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0) return FSB_ERR_BAD_ARG;
  if (T <= 0) return FSB_OK;
  const long long warps = T * (K / 128);
  const long long blocks = (warps * 32 + 255) / 256;
  quant_act_1x128_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), inv_scale, T, K, ldx, ldq);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// D[M,N] bf16 = block-scaled Aq . Bq^T. K % 128 == 0. b_mn: B stored [K, N] (N contiguous).
FSB_API int fsb_gemm_fp8(const void* aq, const float* sa, const void* bq, const float* sb,
                         long long sb_stride_n, long long sb_stride_k, void* d, int M, int N, int K,
                         long long lda, long long ldb, long long ldd, int b_mn, int* status,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % BK != 0) return FSB_ERR_BAD_ARG;
  if (b_mn && N % 16 != 0) return FSB_ERR_BAD_ARG;
  CUtensorMap map_a, map_b;
  int rc = fsb_make_tmap_2d(&map_a, aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, BK);
  if (rc != FSB_OK) return rc;
  if (!b_mn) rc = fsb_make_tmap_2d(&map_b, bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BN, BK);
  else rc = fsb_make_tmap_2d(&map_b, bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, ldb, BK, BN);
  if (rc != FSB_OK) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return FSB_ERR_BAD_ARG;
  if (g_sms[dev] == 0) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return FSB_ERR_LAUNCH;
    cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < g_sms[dev] ? tiles : g_sms[dev];
  Fp8Args a;
  a.M = M; a.N = N; a.K = K; a.b_mn = b_mn;
  a.sa = sa; a.sb = sb; a.sb_stride_n = sb_stride_n; a.sb_stride_k = sb_stride_k;
  a.d = static_cast<__nv_bfloat16*>(d); a.ldd = ldd; a.status = status;
  gemm_fp8_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(map_a, map_b, a);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
