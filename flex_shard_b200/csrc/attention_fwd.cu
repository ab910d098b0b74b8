// Causal flash-attention forward for sm_100a (head_dim 128, GQA), bf16 in/out.
//
// One CTA owns a 128-row query tile of one head and walks the key/value tiles
// (64 rows each) up to the diagonal:
//   S = Q K^T      tcgen05.mma, A = Q (K-major), B = K (K-major), fp32 in TMEM (double-buffered)
//   P = softmax    4 warps, one TMEM lane (query row) per thread, exp2 with the scale folded in;
//                  the running max is refreshed lazily (only when it grew by more than 2^8)
//   O += P V       tcgen05.mma, A = P (bf16 in swizzled shared memory), B = V (MN-major), fp32 in TMEM
// Two CTAs fit on an SM (112 KB shared memory, 256 TMEM columns each), so one CTA's softmax
// overlaps the other's tensor-core work. Warp roles: 0 = TMA, 1 = MMA + TMEM owner, 2..5 = softmax.
//
// Q, K, V, O are addressed as 2-D [B*S, heads*128] matrices with their own row strides, so they
// may be column slices of one fused QKV projection. LSE is [B, Hq, S] fp32 (natural log).
#include "common.cuh"

namespace {
using namespace fsb;

constexpr int HD = 128;
constexpr int BQ = 128;
constexpr int BKV = 64;
constexpr int Q_BYTES = BQ * HD * 2;        // 32 KB (two 64-wide chunks)
constexpr int KV_BYTES = BKV * HD * 2;      // 16 KB (two 64-wide chunks of 8 KB)
constexpr int P_BYTES = BQ * BKV * 2;       // 16 KB
// No alignment slack: two CTAs must fit in the SM's 228 KB (each also pays 1 KB of reserved
// shared memory), so the dynamic buffer is declared 1024-byte aligned and checked at run time.
constexpr int SMEM_FWD = Q_BYTES + 2 * KV_BYTES + 2 * KV_BYTES + P_BYTES + 128;
constexpr int TMEM_COLS_FWD = 256;          // S0 [0,64) S1 [64,128) O [128,256)
constexpr int THREADS = 192;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct FwdArgs {
  int S, Hq, Hkv;
  float scale_log2;   // softmax_scale * log2(e)
  float scale;        // softmax_scale
  __nv_bfloat16* o;
  long long ldo;
  float* lse;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const FwdArgs args) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(args.status, FSB_ERR_BAD_ARG);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;            // [2][KV_BYTES]
  uint8_t* sV = sK + 2 * KV_BYTES;       // [2][KV_BYTES]
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // x = (head, batch), y = query tile from the bottom of the causal triangle up, so CTAs are
  // handed out longest-job-first.
  const int q_tile = gridDim.y - 1 - blockIdx.y;
  const int h = blockIdx.x % args.Hq, b = blockIdx.x / args.Hq;
  const int hk = h / (args.Hq / args.Hkv);
  const int q0 = q_tile * BQ;
  const int n_kv = (q0 + BQ) / BKV;
  const int row_base = b * args.S;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS_FWD);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_2d(sQ, &map_q, q_full, h * HD, row_base + q0);
      tma_load_2d(sQ + Q_BYTES / 2, &map_q, q_full, h * HD + 64, row_base + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag)) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&k_full[s], KV_BYTES);
        tma_load_2d(sK + s * KV_BYTES, &map_k, &k_full[s], hk * HD, row_base + j * BKV);
        tma_load_2d(sK + s * KV_BYTES + KV_BYTES / 2, &map_k, &k_full[s], hk * HD + 64,
                    row_base + j * BKV);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag)) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&v_full[s], KV_BYTES);
        tma_load_2d(sV + s * KV_BYTES, &map_v, &v_full[s], hk * HD, row_base + j * BKV);
        tma_load_2d(sV + s * KV_BYTES + KV_BYTES / 2, &map_v, &v_full[s], hk * HD + 64,
                    row_base + j * BKV);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop (waits and descriptor arithmetic stay warp-uniform); one elected
    // lane issues the tcgen05 instructions.
    {
      const uint32_t idesc_s = make_idesc(BQ, BKV, 1, 1, 0, 0);
      const uint32_t idesc_o = make_idesc(BQ, HD, 1, 1, 0, 1);
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dp = make_smem_desc_sw128(smem_u32(sP), 16, 1024);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok && lane == 0) {
        atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
        *abort_flag = 1;
      }
      for (int j = 0; j <= n_kv && ok; ++j) {
        if (j < n_kv) {
          const int s = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (!mbar_wait(&k_full[s], ph, abort_flag) || !mbar_wait(&s_empty[s], ph ^ 1, abort_flag)) {
            if (lane == 0) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
              *abort_flag = 1;
            }
            break;
          }
          tc_fence_after();
          const uint64_t dk = make_smem_desc_sw128(smem_u32(sK + s * KV_BYTES), 16, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
              const uint32_t qo = ((k >> 2) * (Q_BYTES / 2) + (k & 3) * 32) >> 4;
              const uint32_t ko = ((k >> 2) * (KV_BYTES / 2) + (k & 3) * 32) >> 4;
              umma_f16(tmem_base + s * BKV, dq + qo, dk + ko, idesc_s, k != 0);
            }
            umma_commit(&k_empty[s]);
            umma_commit(&s_full[s]);
          }
          __syncwarp();
        }
        if (j > 0) {
          const int jj = j - 1;
          const int s = jj & 1;
          const uint32_t ph = (jj >> 1) & 1;
          if (!mbar_wait(p_full, jj & 1, abort_flag) || !mbar_wait(&v_full[s], ph, abort_flag)) {
            if (lane == 0) {
              atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_FULL);
              *abort_flag = 1;
            }
            break;
          }
          tc_fence_after();
          // A = P: K-major, 16 kv per step = 32 B inside the 128-byte row.
          // B = V: MN-major, d chunks 8 KB apart (LBO), 8-kv groups 1 KB apart (SBO), 16 kv = 2 KB.
          const uint64_t dv = make_smem_desc_sw128(smem_u32(sV + s * KV_BYTES), KV_BYTES / 2, 1024);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
              umma_f16(tmem_o, dp + ((k * 32) >> 4), dv + ((k * 2048) >> 4), idesc_o, (jj | k) != 0);
            umma_commit(&v_empty[s]);
            umma_commit(pv_done);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // row inside the tile == TMEM lane
    const int q_row = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[s], ph, abort_flag)) {
        if (lane == 0) {
          atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(tmem_base + lane_off + s * BKV, r0);
      tmem_ld_32x32(tmem_base + lane_off + s * BKV + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);

      const int kv0 = j * BKV;
      const bool diag = kv0 + BKV - 1 > q0;  // some element of the tile may be masked
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float a = __uint_as_float(r0[i]), c = __uint_as_float(r1[i]);
        if (diag) {
          if (kv0 + i > q_row) a = -INFINITY;
          if (kv0 + 32 + i > q_row) c = -INFINITY;
        }
        r0[i] = __float_as_uint(a);
        r1[i] = __float_as_uint(c);
        mx = fmaxf(mx, fmaxf(a, c));
      }
      const float m_new = fmaxf(m_used, mx);
      const bool need = (j == 0) || ((m_new - m_used) * args.scale_log2 > 8.f);
      const bool warp_need = __any_sync(0xffffffffu, need);
      float alpha = 1.f;
      if (warp_need) {
        if (j > 0) alpha = fast_exp2((m_used - m_new) * args.scale_log2);
        m_used = m_new;
      }
      // Exponentials first (registers only), so they overlap the previous tile's P V product.
      const float mb = m_used * args.scale_log2;
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(r0[2 * i]), args.scale_log2, -mb));
        const float p1 = fast_exp2(fmaf(__uint_as_float(r0[2 * i + 1]), args.scale_log2, -mb));
        const float p2 = fast_exp2(fmaf(__uint_as_float(r1[2 * i]), args.scale_log2, -mb));
        const float p3 = fast_exp2(fmaf(__uint_as_float(r1[2 * i + 1]), args.scale_log2, -mb));
        sum += (p0 + p1) + (p2 + p3);
        pk[i] = pack_bf16x2(p0, p1);
        pk[16 + i] = pack_bf16x2(p2, p3);
      }
      if (j > 0) {
        // P buffer free and O settled: PV of the previous tile has retired.
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag)) {
          if (lane == 0) {
            atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
      }
      if (warp_need && j > 0) {
        l *= alpha;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_o + lane_off + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
              "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
              "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
              ::"r"(tmem_o + lane_off + c0),
              "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
              "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]),
              "r"(o[15]), "r"(o[16]), "r"(o[17]), "r"(o[18]), "r"(o[19]), "r"(o[20]), "r"(o[21]),
              "r"(o[22]), "r"(o[23]), "r"(o[24]), "r"(o[25]), "r"(o[26]), "r"(o[27]), "r"(o[28]),
              "r"(o[29]), "r"(o[30]), "r"(o[31])
              : "memory");
        }
        tmem_st_wait();
      }
      // P row -> shared memory, 16-byte units XOR-swizzled by (row & 7) as the 128B-swizzle MMA expects.
      uint8_t* prow = sP + r * 128;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        uint4 q4 = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        *reinterpret_cast<uint4*>(prow + ((u ^ (r & 7)) << 4)) = q4;
      }
      l += sum;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag)) {
      tc_fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* orow = args.o + static_cast<long long>(row_base + q_row) * args.ldo + h * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_off + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 pk;
          pk.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
          pk.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
          pk.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
          pk.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c0 + i) = pk;
        }
      }
      args.lse[(static_cast<long long>(b) * args.Hq + h) * args.S + q_row] =
          m_used * args.scale + logf(l);
    } else if (ok && lane == 0) {
      atomicExch(args.status, FSB_ERR_WAIT_TIMEOUT_TMEM_FULL);
      *abort_flag = 1;
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
    tmem_dealloc(tmem_base, TMEM_COLS_FWD);
  }
}

}  // namespace

// q/k/v/o: bf16 matrices [B*S, heads*128] with row strides ldq/ldk/ldv/ldo (elements).
// lse: fp32 [B, Hq, S]. S must be a multiple of 128; Hq a multiple of Hkv.
FSB_API int fsb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S,
                         int Hq, int Hkv, long long ldq, long long ldk, long long ldv, long long ldo,
                         float softmax_scale, int* status, cudaStream_t stream) {
  if (S % BQ != 0 || Hq % Hkv != 0 || B <= 0 || (ldo % 8) != 0) return FSB_ERR_BAD_ARG;
  CUtensorMap mq, mk, mv;
  int rc = fsb_make_tmap_2d(&mq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(B) * S,
                            static_cast<uint64_t>(Hq) * HD, ldq, BQ, 64);
  if (rc != FSB_OK) return rc;
  rc = fsb_make_tmap_2d(&mk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(B) * S,
                        static_cast<uint64_t>(Hkv) * HD, ldk, BKV, 64);
  if (rc != FSB_OK) return rc;
  rc = fsb_make_tmap_2d(&mv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(B) * S,
                        static_cast<uint64_t>(Hkv) * HD, ldv, BKV, 64);
  if (rc != FSB_OK) return rc;
  if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_FWD) !=
      cudaSuccess)
    return FSB_ERR_LAUNCH;
  FwdArgs a;
  a.S = S; a.Hq = Hq; a.Hkv = Hkv;
  a.scale = softmax_scale;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.o = static_cast<__nv_bfloat16*>(o);
  a.ldo = ldo;
  a.lse = lse;
  a.status = status;
  dim3 grid(Hq * B, S / BQ, 1);
  attn_fwd_kernel<<<grid, THREADS, SMEM_FWD, stream>>>(mq, mk, mv, a);
  return cudaGetLastError() == cudaSuccess ? FSB_OK : FSB_ERR_LAUNCH;
}
