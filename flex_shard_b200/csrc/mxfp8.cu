// MXFP8 (e4m3 data, one power-of-two e8m0 scale per 32 elements) for sm_100a:
//   * weight quantiser: one scale per 32x32 tile, so the same data serves a product that contracts
//     over the columns (forward) and one that contracts over the rows (input gradient); the tile
//     exponents are expanded into one scale tensor per orientation;
//   * activation quantiser: one scale per (row, 32-column group);
//   * block-scaled GEMM: tcgen05.mma kind::mxf8f6f4.block_scale. The tensor core applies the
//     scales itself: they sit in TMEM next to the accumulators, copied there from shared memory
//     with tcgen05.cp by the MMA-issuing thread right before the four 32-deep MMAs of a stage.
//
// Scale exponent ("round up" rule): the smallest power of two s with amax / s <= 448, stored as
// the biased byte e = log2(s) + 127 (0 when the group is all zeros); q = round_to_e4m3(x / s).
//
// Scale tensors use the tensor core's block layout: rows in blocks of 128, 32-element groups in
// blocks of 4; block (rb, gb) is 512 contiguous bytes at ((rb * n_gb + gb) * 512) with the byte of
// (row r, group g) at (r % 32) * 16 + (r / 32) * 4 + g. One block is exactly what one 128-row
// operand tile needs for one 128-deep stage, so a stage's scales arrive with one 512-byte bulk copy.
#include "common.cuh"
#include <cuda_fp8.h>

namespace {
using namespace fsb;

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

// biased exponent of the smallest power of two >= amax / 448
__device__ __forceinline__ uint32_t e8m0_round_up(float amax) {
  const float v = amax * (1.f / 448.f);
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = (bits >> 23) & 0xffu;
  if ((bits & 0x7fffffu) != 0 && e < 254u) e += 1;
  return amax > 0.f ? (e > 254u ? 254u : e) : 0u;
}
__device__ __forceinline__ float e8m0_inv(uint32_t e) {   // 2^(127 - e), finite for every e in [0, 254]
  return __uint_as_float(e == 254u ? 0x00400000u : ((254u - e) << 23));
}
__device__ __forceinline__ long long blocked_offset(long long r, int g, int n_gb) {
  return ((r >> 7) * n_gb + (g >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (g & 3);
}

// ------------------------------------------------------------------ weight quantiser (32x32 tiles)
// grid = (ceil(cols/32), ceil(rows/32)), 128 threads: thread t owns row t/4 and 8 columns.
__global__ void __launch_bounds__(128)
mx_quant_weight_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, uint8_t* __restrict__ tile_exp,
                       int rows, int cols, long long ldw, long long ldq, int exp_cols) {
  __shared__ float red[4];
  const int r = blockIdx.y * 32 + (threadIdx.x >> 2);
  const int c0 = blockIdx.x * 32 + (threadIdx.x & 3) * 8;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = (r < rows && c0 + j < cols) ? __bfloat162float(w[r * ldw + c0 + j]) : 0.f;
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const uint32_t e = e8m0_round_up(amax);
  if (threadIdx.x == 0) tile_exp[blockIdx.y * exp_cols + blockIdx.x] = static_cast<uint8_t>(e);
  const float inv = e8m0_inv(e);
  if (r < rows) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < cols)
        q[r * ldq + c0 + j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3));
  }
}

// Tile exponents [ceil(rows/32), ceil(cols/32)] -> blocked scales for the operand [rows, cols]
// (transpose == 0: groups run along the columns) or for its transpose [cols, rows] (groups run
// along the rows). Padding rows / groups get exponent 127 (scale 1).
__global__ void mx_expand_scales_kernel(const uint8_t* __restrict__ tile_exp, uint8_t* __restrict__ out, int op_rows,
                                        int op_groups, int pad_rows, int pad_groups, int exp_cols, int transpose) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long total = static_cast<long long>(pad_rows) * pad_groups;
  if (i >= total) return;
  const long long r = i / pad_groups;
  const int g = static_cast<int>(i % pad_groups);
  uint8_t e = 127;
  if (r < op_rows && g < op_groups)
    e = transpose ? tile_exp[static_cast<long long>(g) * exp_cols + (r >> 5)] : tile_exp[(r >> 5) * exp_cols + g];
  out[blocked_offset(r, g, pad_groups >> 2)] = e;
}

// ------------------------------------------------------------------ activation quantiser (1x32 groups)
// One warp per (row, 128-column span): lane l owns 4 columns, 8 lanes share a scale.
__global__ void mx_quant_act_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                    uint8_t* __restrict__ scales, long long T, int K, long long ldx, long long ldq,
                                    int n_gb) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int spans = K / 128;
  if (w >= T * spans) return;
  const long long row = w / spans;
  const int sp = static_cast<int>(w % spans);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + row * ldx + sp * 128 + lane * 4);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(b2[0]), b = __bfloat1622float2(b2[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const uint32_t e = e8m0_round_up(amax);
  const float inv = e8m0_inv(e);
  if ((lane & 7) == 0) scales[blocked_offset(row, sp * 4 + (lane >> 3), n_gb)] = static_cast<uint8_t>(e);
  uint8_t o[4];
  o[0] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(a.x * inv, __NV_SATFINITE, __NV_E4M3));
  o[1] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(a.y * inv, __NV_SATFINITE, __NV_E4M3));
  o[2] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(b.x * inv, __NV_SATFINITE, __NV_E4M3));
  o[3] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(b.y * inv, __NV_SATFINITE, __NV_E4M3));
  *reinterpret_cast<uint32_t*>(q + row * ldq + sp * 128 + lane * 4) = *reinterpret_cast<const uint32_t*>(o);
}

// ------------------------------------------------------------------ transposed-use quantiser (32x1 groups)
// For products that contract over the rows of x (weight gradients): one scale per (32-row group,
// column). The data keeps its row-major layout; the scales are those of the operand x^T, i.e. blocked
// with "rows" = columns of x and groups = 32-row groups of x. grid = (K/128, T/32), 128 threads:
// thread t owns column 128*bx + t over the 32 rows of the group (loads and byte stores are coalesced).
__global__ void __launch_bounds__(128)
mx_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ scales,
                     long long T, int K, long long ldx, long long ldq, int n_gb) {
  const int col = blockIdx.x * 128 + threadIdx.x;
  const long long r0 = static_cast<long long>(blockIdx.y) * 32;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = (r0 + i < T) ? __bfloat162float(x[(r0 + i) * ldx + col]) : 0.f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  const uint32_t e = e8m0_round_up(amax);
  const float inv = e8m0_inv(e);
  scales[blocked_offset(col, static_cast<int>(blockIdx.y), n_gb)] = static_cast<uint8_t>(e);
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (r0 + i < T)
      q[(r0 + i) * ldq + col] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3));
}

// ------------------------------------------------------------------ block-scaled GEMM
constexpr int BM = 128, BN = 128, BK = 128;  // BK bytes == elements (fp8)
constexpr int STAGES = 6;
constexpr int A_STAGE = BM * BK, B_STAGE = BN * BK, SF_BYTES = 512;
constexpr int STAGE_BYTES = A_STAGE + B_STAGE + 2 * SF_BYTES;   // 33 KB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int NUM_THREADS = 192;   // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int TMEM_COLS = 512;     // two 128-column accumulators + two sets of (4 + 4) scale columns
constexpr int SF_COL0 = 256;

struct MxArgs {
  int M, N, K;
  int a_mn, b_mn;
  const uint8_t* sfa;   // blocked scales of A: [ceil(M/128)][K/128][512]
  const uint8_t* sfb;   // blocked scales of B: [ceil(N/128)][K/128][512]
  void* d;
  long long ldd;
  int d_fp32;
  int* status;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, repeated in all four lane quarters
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Unswizzled K-major descriptor: 8-row groups of 16-byte rows are 128 bytes apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // SBO
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// e4m3 x e4m3, e8m0 scales; sf_id selects which of a scale word's four bytes (which 32-deep group
// of the stage) this MMA uses.
__device__ __forceinline__ uint32_t make_idesc_mx(uint32_t m, uint32_t n, uint32_t a_mn, uint32_t b_mn, uint32_t sf_id) {
  return (sf_id << 4) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf_id << 29);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const MxArgs args) {
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
      mbar_init(&tmem_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
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
          uint8_t* ssf = sb + B_STAGE;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          if (!args.a_mn) tma_load_2d(sa, &map_a, &full_bar[s], kb * BK, tm * BM);
          else tma_load_2d(sa, &map_a, &full_bar[s], tm * BM, kb * BK);  // [K rows][128 M bytes]
          if (!args.b_mn) tma_load_2d(sb, &map_b, &full_bar[s], kb * BK, tn * BN);
          else tma_load_2d(sb, &map_b, &full_bar[s], tn * BN, kb * BK);  // [K rows][128 N bytes]
          bulk_load_1d(ssf, args.sfa + (static_cast<long long>(tm) * num_kb + kb) * SF_BYTES, SF_BYTES, &full_bar[s]);
          bulk_load_1d(ssf + SF_BYTES, args.sfb + (static_cast<long long>(tn) * num_kb + kb) * SF_BYTES, SF_BYTES,
                       &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop; one elected lane issues the tcgen05 instructions.
    // K-major: 32 elements (bytes) per MMA inside the 128-byte row. MN-major B: one 128-wide
    // N group, 8-deep K groups 1 KB apart, 32 K = 4 groups = 4 KB per MMA.
    const uint32_t a_kstep = (args.a_mn ? 4096u : 32u) >> 4, b_kstep = (args.b_mn ? 4096u : 32u) >> 4;
    const uint32_t a_mn = args.a_mn ? 1u : 0u, b_mn = args.b_mn ? 1u : 0u;
    uint32_t it = 0, local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      ++local_tile;
      if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
        if (lane == 0) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph, abort_flag)) {
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
        const uint32_t ssf = sa + A_STAGE + B_STAGE;
        const uint32_t tsfa = tmem_base + SF_COL0 + (it & 1) * 8, tsfb = tsfa + 4;
        if (elect_one()) {
          tmem_cp_32x128b_x4(tsfa, make_sf_desc(ssf));
          tmem_cp_32x128b_x4(tsfb, make_sf_desc(ssf + SF_BYTES));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_mxf8(tmem_base + acc * BN, da + k * a_kstep, db + k * b_kstep, make_idesc_mx(BM, BN, a_mn, b_mn, k), tsfa, tsfb,
                      (kb | k) != 0);
          umma_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (ok) {
        if (elect_one()) umma_commit(&tmem_full[acc]);
        __syncwarp();
      }
    }
  } else {
    const int quarter = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const long long row = static_cast<long long>(tm) * BM + quarter * 32 + lane;
      const bool row_ok = row < args.M;
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      ++local_tile;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col = tn * BN + c0;
        if (col >= args.N) break;
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_off + acc * BN + c0, v);
        tmem_ld_wait();
        if (!row_ok) continue;
        const int ncols = min(32, args.N - col);
        if (args.d_fp32) {
          float* dp = static_cast<float*>(args.d) + row * args.ldd + col;
          for (int i = 0; i < ncols; ++i) dp[i] = __uint_as_float(v[i]);
        } else {
          __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(args.d) + row * args.ldd + col;
          if (ncols == 32 && (args.ldd % 8) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
              *reinterpret_cast<uint4*>(dp + i) = o;
            }
          } else {
            for (int i = 0; i < ncols; ++i) dp[i] = __float2bfloat16(__uint_as_float(v[i]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int g_sms[64] = {0};
}  // namespace

// w: bf16 [rows, cols]; q: e4m3 [rows, cols]; tile_exp: uint8 [ceil(rows/32), ceil(cols/32)].
FSB_API int fsb_mx_quant_weight(const void* w, void* q, void* tile_exp, int rows, int cols, long long ldw,
                                long long ldq, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return FSB_OK;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  mx_quant_weight_kernel<<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q),
                                                   static_cast<uint8_t*>(tile_exp), rows, cols, ldw, ldq,
                                                   (cols + 31) / 32);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// Blocked scales of the operand [rows, cols] (transpose == 0) or [cols, rows] (transpose == 1) from
// the tile exponents of a [rows, cols] weight. out: pad128(op rows) * pad4(ceil(op cols / 32)) bytes.
FSB_API int fsb_mx_expand_scales(const void* tile_exp, void* out, int rows, int cols, int transpose,
                                 cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return FSB_OK;
  const int op_rows = transpose ? cols : rows;
  const int op_groups = ((transpose ? rows : cols) + 31) / 32;
  const int pad_rows = (op_rows + 127) / 128 * 128, pad_groups = (op_groups + 3) / 4 * 4;
  const long long total = static_cast<long long>(pad_rows) * pad_groups;
  mx_expand_scales_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(tile_exp), static_cast<uint8_t*>(out), op_rows, op_groups, pad_rows, pad_groups,
      (cols + 31) / 32, transpose);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// x: bf16 [T, K], K % 128 == 0; q: e4m3 [T, K]; scales: blocked, pad128(T) * (K/32) bytes (rows past T
// are not written: allocate zeroed or ignore them, they only feed output rows that are masked).
FSB_API int fsb_mx_quant_act(const void* x, void* q, void* scales, long long T, int K, long long ldx, long long ldq,
                             cudaStream_t stream) {
  if (K % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0) return FSB_ERR_BAD_ARG;
  if (T <= 0) return FSB_OK;
  const long long warps = T * (K / 128);
  mx_quant_act_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(scales), T, K, ldx, ldq,
      K / 128);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// x: bf16 [T, K] with T % 128 == 0 and K % 128 == 0; q: e4m3 [T, K] (same layout); scales: blocked scales of
// the operand x^T ([K rows, T/32 groups]): K * (T/32) bytes.
FSB_API int fsb_mx_quant_rows(const void* x, void* q, void* scales, long long T, int K, long long ldx, long long ldq,
                              cudaStream_t stream) {
  if (K % 128 != 0 || T % 128 != 0) return FSB_ERR_BAD_ARG;
  if (T <= 0) return FSB_OK;
  dim3 grid(K / 128, static_cast<unsigned>(T / 32));
  mx_quant_rows_kernel<<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q),
                                                 static_cast<uint8_t*>(scales), T, K, ldx, ldq,
                                                 static_cast<int>(T / 128));
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}

// D[M,N] = (Aq * 2^sfa) . (Bq * 2^sfb)^T with K % 128 == 0. A: e4m3 [M, K] (a_mn == 0) or [K, M]
// (a_mn == 1: M contiguous, M % 16 == 0). B: e4m3 [N, K] (b_mn == 0) or [K, N] (b_mn == 1: N contiguous,
// N % 16 == 0). sfa / sfb: blocked scales of the
// operands as the GEMM sees them ([M, K] and [N, K]).
FSB_API int fsb_gemm_mxfp8(const void* aq, const void* sfa, const void* bq, const void* sfb, void* d, int M, int N,
                           int K, long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int d_fp32,
                           int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % BK != 0) return FSB_ERR_BAD_ARG;
  if ((b_mn && N % 16 != 0) || (a_mn && M % 16 != 0)) return FSB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb)) & 15) return FSB_ERR_BAD_ARG;
  CUtensorMap map_a, map_b;
  int rc;
  if (!a_mn) rc = fsb_make_tmap_2d(&map_a, aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, BM, BK);
  else rc = fsb_make_tmap_2d(&map_a, aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, lda, BK, BM);
  if (rc != FSB_OK) return rc;
  if (!b_mn) rc = fsb_make_tmap_2d(&map_b, bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BN, BK);
  else rc = fsb_make_tmap_2d(&map_b, bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, ldb, BK, BN);
  if (rc != FSB_OK) return rc;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return FSB_ERR_BAD_ARG;
  if (g_sms[dev] == 0) {
    if (cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return FSB_ERR_LAUNCH;
    cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < g_sms[dev] ? tiles : g_sms[dev];
  MxArgs a;
  a.M = M; a.N = N; a.K = K; a.a_mn = a_mn; a.b_mn = b_mn;
  a.sfa = static_cast<const uint8_t*>(sfa); a.sfb = static_cast<const uint8_t*>(sfb);
  a.d = d; a.ldd = ldd; a.d_fp32 = d_fp32; a.status = status;
  gemm_mxfp8_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(map_a, map_b, a);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
